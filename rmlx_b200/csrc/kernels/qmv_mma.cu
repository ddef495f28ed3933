// 4-bit (MLX affine, group 64) matrix-vector products for decode: bulk-copy-fed, tensor-core
// multiplied.
//
// Two costs dominate a Q4 mat-vec on this GPU, and neither is DRAM bandwidth: the instructions
// that turn nibbles into numbers, and the load-pipe work of fetching 16 short row segments per
// MMA tile. This kernel family removes both:
//
//  * Weights, scales and biases of a block's rows are brought into shared memory by the TMA unit
//    (cp.async.bulk, one copy per row, completion on an mbarrier). The copies are issued before
//    the block waits on the previous kernel and before it stages the activations, so the whole
//    weight read overlaps everything else, costs no registers and no load instructions.
//  * A nibble becomes an fp16 operand with ONE logic op: OR-ing it into the mantissa of 1024.0
//    gives exactly 1024+q (or 1024+16q for the nibble four bits up, whose activation is staged
//    divided by 16). mma.sync m16n8k16 multiplies with fp32 accumulation, where the 1024*x excess
//    is still exact enough to subtract afterwards; per group
//        sum_k w_k x_k = s * (C - 1024 * sum(staged x)) + b * sum(x).
//    The eight MMA columns carry up to eight activation vectors (decode batch) at no extra cost.
//
// Work split: a block owns 16*TILES output rows, its eight warps split K by groups and are merged
// through shared memory. Lane (g, t) reads 8 bytes (16 weights) of rows g and g+8 per group from
// shared memory (row stride = row bytes + 32, which makes the access conflict-free).
//
// Needs K % 512 == 0 (16-byte granularity of the per-row scale copies); other shapes use the
// scalar kernels of decode_gemv.cu / decode_moe.cu.
//
// Kernels: RMSNorm + projection (+ residual, bf16 or fp32 out), MoE gate/up with SwiGLU, MoE down
// with the routing-weighted sum over slots. Reference counterparts: affine_qmv_fast_* and
// gather_qmv_fast_* (crates/rmlx-core/src/ops/quantized.rs:407,9634), fused with RMSNorm / SwiGLU /
// residual as in crates/rmlx-core/src/ops/fused.rs.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kQThreads = 256;
constexpr int kQWarps = 8;
constexpr int kQMaxTopK = 8;

__device__ int g_qmv_status = 0;  // set to kStatusMbarTimeout if a copy wait ever gives up

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier. Addresses and size are
// multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ------------------------------------------------------------------------------------------------
// Activation staging for one column: K fp16 values in MMA B-fragment order plus, per group, the
// pair (1024 * sum of staged values, sum of true values).
//   fragment unit (G, t, jh) = 8 bytes {b0, b1}, index ((G*4 + t)*4 + jh), jh = 2*j + h,
//   k0 = G*64 + t*16 + j*8:  b0 = (x[k0+2h], x[k0+2h+4]),  b1 = (x[k0+2h+1], x[k0+2h+5]) / 16
// ------------------------------------------------------------------------------------------------
struct QStage {
  static __host__ __device__ size_t frag_bytes(int K) { return size_t(K) * 2 + 16; }  // +16: bank skew
  static __host__ __device__ size_t col_bytes(int K) {
    return (frag_bytes(K) + size_t(K >> 6) * 8 + 15) & ~size_t(15);
  }

  // Writes chunk c (8 values) in fragment order; returns (sum of staged "plain" values, sum of
  // staged "/16" values) as they were rounded to fp16.
  static __device__ __forceinline__ float2 put_chunk(char* col, int c, const float (&f)[8]) {
    const int G = c >> 3, t = (c >> 1) & 3, j = c & 1;
    uint2* u = reinterpret_cast<uint2*>(col) + ((G * 4 + t) * 4 + j * 2);
    const float q = 1.f / 16.f;
    __half2 b00 = __floats2half2_rn(f[0], f[4]), b01 = __floats2half2_rn(f[1] * q, f[5] * q);
    __half2 b10 = __floats2half2_rn(f[2], f[6]), b11 = __floats2half2_rn(f[3] * q, f[7] * q);
    u[0] = make_uint2(*reinterpret_cast<uint32_t*>(&b00), *reinterpret_cast<uint32_t*>(&b01));
    u[1] = make_uint2(*reinterpret_cast<uint32_t*>(&b10), *reinterpret_cast<uint32_t*>(&b11));
    const float2 p0 = __half22float2(b00), p1 = __half22float2(b10);
    const float2 d0 = __half22float2(b01), d1 = __half22float2(b11);
    return make_float2((p0.x + p0.y) + (p1.x + p1.y), (d0.x + d0.y) + (d1.x + d1.y));
  }
  // Stage K bf16 values (optionally times a bf16 weight vector). No block barrier inside: the
  // eight chunks of a group belong to eight neighbouring lanes, so the per-group sums come from
  // three shuffles. Each warp leaves its partial sum of squares of x in red[warp] (when red is
  // given); after ONE __syncthreads() by the caller the staged data, the group sums and red[] are
  // visible, and sum(red[0..7]) is the row's sum of squares. K is a multiple of 256.
  static __device__ void stage(char* col, const __nv_bfloat16* x, const __nv_bfloat16* scale_w,
                               int K, float* red) {
    float2* sums = reinterpret_cast<float2*>(col + frag_bytes(K));
    float ssq = 0.f;
    for (int c = threadIdx.x; c < (K >> 3); c += kQThreads) {   // warp-uniform: K/8 % 32 == 0
      const uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
      float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                    bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq += f[i] * f[i];
      if (scale_w) {
        const uint4 s = *reinterpret_cast<const uint4*>(scale_w + (c << 3));
        f[0] *= bf16lo(s.x); f[1] *= bf16hi(s.x); f[2] *= bf16lo(s.y); f[3] *= bf16hi(s.y);
        f[4] *= bf16lo(s.z); f[5] *= bf16hi(s.z); f[6] *= bf16lo(s.w); f[7] *= bf16hi(s.w);
      }
      float2 s2 = put_chunk(col, c, f);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        s2.x += __shfl_xor_sync(0xffffffffu, s2.x, o);
        s2.y += __shfl_xor_sync(0xffffffffu, s2.y, o);
      }
      if ((c & 7) == 0) sums[c >> 3] = make_float2(1024.f * (s2.x + s2.y), s2.x + 16.f * s2.y);
    }
    if (red) {
      ssq = warp_sum(ssq);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
    }
  }
  static __device__ __forceinline__ float total(const float* red) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kQWarps; ++i) s += red[i];
    return s;
  }
};

// ------------------------------------------------------------------------------------------------
// Shared-memory image of ROWS weight rows: packed words, then scales, then biases, each with its
// own padded row stride.
// ------------------------------------------------------------------------------------------------
struct WTile {
  int K;
  __host__ __device__ int wbytes() const { return K >> 1; }           // packed bytes per row
  __host__ __device__ int sbytes() const { return K >> 5; }           // scale (or bias) bytes per row
  __host__ __device__ int wstride() const { return wbytes() + 32; }   // 32 mod 128: conflict-free LDS.64
  __host__ __device__ int sstride() const { return sbytes() + 16; }
  __host__ __device__ size_t bytes(int rows) const {
    return size_t(rows) * (wstride() + 2 * sstride());
  }
  __device__ char* w(char* base, int row) const { return base + size_t(row) * wstride(); }
  __device__ char* s(char* base, int rows, int row) const {
    return base + size_t(rows) * wstride() + size_t(row) * sstride();
  }
  __device__ char* b(char* base, int rows, int row) const {
    return base + size_t(rows) * (wstride() + sstride()) + size_t(row) * sstride();
  }
  // One lane per row issues that row's three copies. `grow` is the global row index.
  __device__ void issue_row(char* base, int rows, int row, const uint32_t* gw,
                            const __nv_bfloat16* gs, const __nv_bfloat16* gb, size_t grow,
                            uint64_t* bar) const {
    bulk_g2s(w(base, row), gw + grow * size_t(K >> 3), wbytes(), bar);
    bulk_g2s(s(base, rows, row), gs + grow * size_t(K >> 6), sbytes(), bar);
    bulk_g2s(b(base, rows, row), gb + grow * size_t(K >> 6), sbytes(), bar);
  }
};

// Accumulate groups [G0, G1) of one 16-row tile (rows ra = first + g, rb = first + g + 8 of the
// shared-memory image) against the staged columns.
// acc[0..3] = (row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1).
template <int NCOLS>
__device__ __forceinline__ void qmv_tile_groups(const WTile& wt, const char* wbase, int rows,
                                                int row_a, int row_b, const char* stage,
                                                size_t col_stride, int G0, int G1, float (&acc)[4]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int K = wt.K;
  const bool has_col = g < NCOLS;
  const char* mycol = stage + (has_col ? g : 0) * col_stride;
  const size_t fb = QStage::frag_bytes(K);
  const int c0i = 2 * t, c1i = 2 * t + 1;
  const float2* sum0 = reinterpret_cast<const float2*>(stage + (c0i < NCOLS ? c0i : 0) * col_stride + fb);
  const float2* sum1 = reinterpret_cast<const float2*>(stage + (c1i < NCOLS ? c1i : 0) * col_stride + fb);
  const char* wa_row = wbase + size_t(row_a) * wt.wstride() + t * 8;
  const char* wb_row = wbase + size_t(row_b) * wt.wstride() + t * 8;
  const __nv_bfloat16* sa = reinterpret_cast<const __nv_bfloat16*>(
      wbase + size_t(rows) * wt.wstride() + size_t(row_a) * wt.sstride());
  const __nv_bfloat16* sb = reinterpret_cast<const __nv_bfloat16*>(
      wbase + size_t(rows) * wt.wstride() + size_t(row_b) * wt.sstride());
  const size_t bias_off = size_t(rows) * wt.sstride() / 2;  // in bf16 elements
#pragma unroll 2
  for (int G = G0; G < G1; ++G) {
    const uint2 wa = *reinterpret_cast<const uint2*>(wa_row + G * 32);
    const uint2 wb = *reinterpret_cast<const uint2*>(wb_row + G * 32);
    uint4 f01 = make_uint4(0, 0, 0, 0), f23 = f01;
    if (has_col) {
      const uint4* fp = reinterpret_cast<const uint4*>(mycol) + (G * 4 + t) * 2;
      f01 = fp[0]; f23 = fp[1];
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const uint32_t a = wa.x, b = wb.x, a8 = a >> 8, b8 = b >> 8;
      mma_f16_16816(c, (a & 0x000f000fu) | 0x64006400u, (b & 0x000f000fu) | 0x64006400u,
                    (a & 0x00f000f0u) | 0x64006400u, (b & 0x00f000f0u) | 0x64006400u, f01.x, f01.y);
      mma_f16_16816(c, (a8 & 0x000f000fu) | 0x64006400u, (b8 & 0x000f000fu) | 0x64006400u,
                    (a8 & 0x00f000f0u) | 0x64006400u, (b8 & 0x00f000f0u) | 0x64006400u, f01.z, f01.w);
    }
    {
      const uint32_t a = wa.y, b = wb.y, a8 = a >> 8, b8 = b >> 8;
      mma_f16_16816(c, (a & 0x000f000fu) | 0x64006400u, (b & 0x000f000fu) | 0x64006400u,
                    (a & 0x00f000f0u) | 0x64006400u, (b & 0x00f000f0u) | 0x64006400u, f23.x, f23.y);
      mma_f16_16816(c, (a8 & 0x000f000fu) | 0x64006400u, (b8 & 0x000f000fu) | 0x64006400u,
                    (a8 & 0x00f000f0u) | 0x64006400u, (b8 & 0x00f000f0u) | 0x64006400u, f23.z, f23.w);
    }
    const float s_a = __bfloat162float(sa[G]), s_b = __bfloat162float(sb[G]);
    const float b_a = __bfloat162float(sa[bias_off + G]), b_b = __bfloat162float(sb[bias_off + G]);
    const float2 s0 = sum0[G], s1 = sum1[G];   // (1024*sum staged, sum true)
    acc[0] += s_a * (c[0] - s0.x) + b_a * s0.y;
    acc[1] += s_a * (c[1] - s1.x) + b_a * s1.y;
    acc[2] += s_b * (c[2] - s0.x) + b_b * s0.y;
    acc[3] += s_b * (c[3] - s1.x) + b_b * s1.y;
  }
}

__device__ __forceinline__ void warp_group_range(int ng, int warp, int& G0, int& G1) {
  const int per = (ng + kQWarps - 1) / kQWarps;
  G0 = min(ng, warp * per);
  G1 = min(ng, G0 + per);
}

// Bounded wait for the block's weight image; every thread observes the completed phase itself,
// which also makes the async-proxy writes visible to it.
__device__ __forceinline__ void wait_weights(uint64_t* bar, uint32_t parity) {
  bool ok = false;
  for (uint32_t i = 0; i < kMbarPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) { ok = true; break; }
  }
  if (!ok) atomicExch(&g_qmv_status, kStatusMbarTimeout);
}

// ------------------------------------------------------------------------------------------------
// out[b, n] = residual[b, n] + inv_rms[b] * sum_k W[n,k] * (x[b,k] * g[k])
// ------------------------------------------------------------------------------------------------
template <int NCOLS, int TILES, bool OUT_F32>
__global__ void __launch_bounds__(kQThreads)
rms_qmv_mma_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ scales,
                   const __nv_bfloat16* __restrict__ biases, const __nv_bfloat16* __restrict__ x,
                   int x_stride, const __nv_bfloat16* __restrict__ norm_w, float eps,
                   const __nv_bfloat16* __restrict__ residual, int res_stride,
                   void* __restrict__ out, int out_stride, int N, int K) {
  constexpr int ROWS = 16 * TILES;
  extern __shared__ __align__(128) char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ float red[NCOLS][kQWarps];
  __shared__ float part[kQWarps][TILES][16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const WTile wt{K};
  char* wimg = smem;
  char* xst = smem + ((wt.bytes(ROWS) + 127) & ~size_t(127));
  const size_t cstride = QStage::col_bytes(K);
  const int row0 = blockIdx.x * ROWS;

  // Warp 0 alone sets up the barrier and issues the copies; everyone else first meets the barrier
  // after the block-wide sync below.
  if (warp == 0) {
    if (lane == 0) {
      mbar_init(&bar, 1);
      fence_mbar_init();
      mbar_arrive_expect_tx(&bar, uint32_t(ROWS) * (wt.wbytes() + 2 * wt.sbytes()));
    }
    __syncwarp();
    for (int r = lane; r < ROWS; r += 32)
      wt.issue_row(wimg, ROWS, r, w, scales, biases, size_t(min(row0 + r, N - 1)), &bar);
  }
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
#pragma unroll
  for (int b = 0; b < NCOLS; ++b)
    QStage::stage(xst + b * cstride, x + size_t(b) * x_stride, norm_w, K, red[b]);
  __syncthreads();
  float inv_rms[NCOLS];
#pragma unroll
  for (int b = 0; b < NCOLS; ++b)
    inv_rms[b] = norm_w ? rsqrtf(QStage::total(red[b]) / float(K) + eps) : 1.f;
  wait_weights(&bar, 0);
  int G0, G1;
  warp_group_range(K >> 6, warp, G0, G1);
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    qmv_tile_groups<NCOLS>(wt, wimg, ROWS, tl * 16 + g, tl * 16 + g + 8, xst, cstride, G0, G1, acc);
    part[warp][tl][g][2 * t] = acc[0]; part[warp][tl][g][2 * t + 1] = acc[1];
    part[warp][tl][g + 8][2 * t] = acc[2]; part[warp][tl][g + 8][2 * t + 1] = acc[3];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ROWS * NCOLS; i += kQThreads) {
    const int col = i / ROWS, rr = i % ROWS;
    const int n = row0 + rr;
    if (n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int wv = 0; wv < kQWarps; ++wv) v += part[wv][rr >> 4][rr & 15][col];
    float ir = inv_rms[0];
#pragma unroll
    for (int b = 1; b < NCOLS; ++b) ir = (col == b) ? inv_rms[b] : ir;
    v *= ir;
    if (residual) v += __bfloat162float(residual[size_t(col) * res_stride + n]);
    if (OUT_F32) reinterpret_cast<float*>(out)[size_t(col) * out_stride + n] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[size_t(col) * out_stride + n] = __float2bfloat16_rn(v);
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// MoE gate/up + SwiGLU per (token, slot). Tile tl holds gate rows i0 + 8*tl + [0,8) in image rows
// 16*tl + [0,8) and the matching up rows in 16*tl + [8,16), so a SwiGLU pair meets in one lane.
// grid = (I / (8*TILES), tokens*top_k).
// ------------------------------------------------------------------------------------------------
template <int TILES>
__global__ void __launch_bounds__(kQThreads)
moe_gate_up_q4_mma_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ scales,
                          const __nv_bfloat16* __restrict__ biases,
                          const __nv_bfloat16* __restrict__ x, int x_stride,
                          const __nv_bfloat16* __restrict__ norm_w, float eps,
                          const int* __restrict__ topk_idx, __nv_bfloat16* __restrict__ act,
                          int act_stride, int I, int K, int top_k, int expert_base,
                          int experts_local) {
  constexpr int ROWS = 16 * TILES;
  extern __shared__ __align__(128) char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ float red[kQWarps];
  __shared__ float part[kQWarps][TILES][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int pair = blockIdx.y, b = pair / top_k;
  const WTile wt{K};
  char* wimg = smem;
  char* xst = smem + ((wt.bytes(ROWS) + 127) & ~size_t(127));
  const size_t cstride = QStage::col_bytes(K);
  const int i0 = blockIdx.x * 8 * TILES;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();   // the expert index comes from the router kernel
  const int e = topk_idx[pair] - expert_base;
  if (e < 0 || e >= experts_local) return;
  if (warp == 0) {
    if (lane == 0) {
      mbar_init(&bar, 1);
      fence_mbar_init();
      mbar_arrive_expect_tx(&bar, uint32_t(ROWS) * (wt.wbytes() + 2 * wt.sbytes()));
    }
    __syncwarp();
    const size_t ebase = size_t(e) * 2 * I;
    for (int r = lane; r < ROWS; r += 32) {
      const int tl = r >> 4, rr = r & 15;
      const int i = min(i0 + tl * 8 + (rr & 7), I - 1);
      wt.issue_row(wimg, ROWS, r, w, scales, biases, ebase + (rr < 8 ? i : I + i), &bar);
    }
  }
  QStage::stage(xst, x + size_t(b) * x_stride, norm_w, K, red);
  __syncthreads();
  const float inv_rms_s = norm_w ? rsqrtf(QStage::total(red) / float(K) + eps) : 1.f;
  wait_weights(&bar, 0);
  int G0, G1;
  warp_group_range(K >> 6, warp, G0, G1);
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    qmv_tile_groups<1>(wt, wimg, ROWS, tl * 16 + g, tl * 16 + g + 8, xst, cstride, G0, G1, acc);
    if (t == 0) { part[warp][tl][g] = acc[0]; part[warp][tl][g + 8] = acc[2]; }
  }
  __syncthreads();
  if (threadIdx.x < TILES * 8) {
    const int tl = threadIdx.x >> 3, gg = threadIdx.x & 7;
    const int i = i0 + tl * 8 + gg;
    if (i < I) {
      float gt = 0.f, up = 0.f;
#pragma unroll
      for (int wv = 0; wv < kQWarps; ++wv) { gt += part[wv][tl][gg]; up += part[wv][tl][gg + 8]; }
      gt *= inv_rms_s; up *= inv_rms_s;
      act[size_t(pair) * act_stride + i] = __float2bfloat16_rn(gt / (1.f + __expf(-gt)) * up);
    }
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// MoE down: out[b, n] = residual[b, n] + sum_slot wts[b, slot] * Wd[e_slot][n, :] . act[b, slot, :]
// grid = (N / 16, tokens). All local slots' weight rows are in flight at once.
// ------------------------------------------------------------------------------------------------
template <bool OUT_F32>
__global__ void __launch_bounds__(kQThreads)
moe_down_q4_mma_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ scales,
                       const __nv_bfloat16* __restrict__ biases,
                       const __nv_bfloat16* __restrict__ act, int act_stride,
                       const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                       const __nv_bfloat16* __restrict__ residual, int res_stride,
                       void* __restrict__ out, int out_stride, int N, int I, int top_k,
                       int expert_base, int experts_local) {
  extern __shared__ __align__(128) char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_e[kQMaxTopK];
  __shared__ float s_w[kQMaxTopK];
  __shared__ float part[kQWarps][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.y;
  const WTile wt{I};
  const size_t img = (wt.bytes(16) + 127) & ~size_t(127);
  char* xst = smem + img * top_k;
  const size_t cstride = QStage::col_bytes(I);
  const int row0 = blockIdx.x * 16;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  // Every thread reads the (few) routing entries itself: no barrier before the copies go out.
  int my_e[kQMaxTopK];
#pragma unroll
  for (int s = 0; s < kQMaxTopK; ++s) {
    int e = -1;
    if (s < top_k) {
      e = topk_idx[b * top_k + s] - expert_base;
      if (e < 0 || e >= experts_local) e = -1;
    }
    my_e[s] = e;
  }
  if (warp == 0) {
    int nlocal = 0;
#pragma unroll
    for (int s = 0; s < kQMaxTopK; ++s) nlocal += my_e[s] >= 0;
    if (lane == 0) {
      mbar_init(&bar, 1);
      fence_mbar_init();
      mbar_arrive_expect_tx(&bar, uint32_t(nlocal) * 16u * (wt.wbytes() + 2 * wt.sbytes()));
    }
    __syncwarp();
#pragma unroll
    for (int s = 0; s < kQMaxTopK; ++s) {
      if (my_e[s] >= 0 && lane < 16)
        wt.issue_row(smem + img * s, 16, lane, w, scales, biases,
                     size_t(my_e[s]) * N + min(row0 + lane, N - 1), &bar);
    }
  }
#pragma unroll
  for (int s = 0; s < kQMaxTopK; ++s) {
    if (my_e[s] >= 0)
      QStage::stage(xst + s * cstride, act + size_t(b * top_k + s) * act_stride, nullptr, I, nullptr);
    if (threadIdx.x == s) {
      s_e[s] = my_e[s];
      s_w[s] = my_e[s] >= 0 ? topk_w[b * top_k + s] : 0.f;
    }
  }
  __syncthreads();
  wait_weights(&bar, 0);
  int G0, G1;
  warp_group_range(I >> 6, warp, G0, G1);
  float tot0 = 0.f, tot2 = 0.f;
  for (int s = 0; s < top_k; ++s) {
    if (s_e[s] < 0) continue;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    qmv_tile_groups<1>(wt, smem + img * s, 16, g, g + 8, xst + s * cstride, cstride, G0, G1, acc);
    tot0 = fmaf(s_w[s], acc[0], tot0);
    tot2 = fmaf(s_w[s], acc[2], tot2);
  }
  if (t == 0) { part[warp][g] = tot0; part[warp][g + 8] = tot2; }
  __syncthreads();
  if (threadIdx.x < 16) {
    const int n = row0 + threadIdx.x;
    if (n < N) {
      float v = 0.f;
#pragma unroll
      for (int wv = 0; wv < kQWarps; ++wv) v += part[wv][threadIdx.x];
      if (residual) v += __bfloat162float(residual[size_t(b) * res_stride + n]);
      if (OUT_F32) reinterpret_cast<float*>(out)[size_t(b) * out_stride + n] = v;
      else reinterpret_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n] = __float2bfloat16_rn(v);
    }
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// Grouped narrow-M expert projections: activation rows sorted by expert (rows offsets[e] ..
// offsets[e+1] of x belong to local expert e), a handful of rows per expert (decode batches of
// 16-64 tokens spread over a hundred experts). Block (row tile, expert) brings its weight rows
// into shared memory ONCE and multiplies them with all of the expert's rows, NCOLS at a time; an
// expert without rows costs an early exit. A 128-row tensor-core tile per expert would spend the
// same dequantisation work per weight on rows that do not exist.
//   SWIGLU: weights [E, 2 I, K] (gate rows, then up rows), out[r, i] = silu(gate) * up, N = I;
//           tile tl holds gate rows i0 + 8 tl + [0, 8) in image rows 16 tl + [0, 8) and the
//           matching up rows in 16 tl + [8, 16).
//   else:   weights [E, N, K], out[r, n] = W[e][n, :] . x[r, :].
// grid = (row tiles, local experts).
// ------------------------------------------------------------------------------------------------
template <int NCOLS, int TILES, bool SWIGLU>
__global__ void __launch_bounds__(kQThreads)
grouped_qmv_mma_kernel(const uint32_t* __restrict__ w, const __nv_bfloat16* __restrict__ scales,
                       const __nv_bfloat16* __restrict__ biases, const __nv_bfloat16* __restrict__ x,
                       int x_stride, const int* __restrict__ offsets, __nv_bfloat16* __restrict__ out,
                       int out_stride, int N, int K) {
  constexpr int ROWS = 16 * TILES;
  extern __shared__ __align__(128) char smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ float part[kQWarps][TILES][16][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int e = blockIdx.y;
  const WTile wt{K};
  char* wimg = smem;
  char* xst = smem + ((wt.bytes(ROWS) + 127) & ~size_t(127));
  const size_t cstride = QStage::col_bytes(K);
  const int first = blockIdx.x * (SWIGLU ? 8 * TILES : ROWS);   // first output row / first gate row
  pdl_launch_dependents();
  pdl_wait();                       // the offsets come from the routing kernel
  const int r0 = offsets[e], r1 = offsets[e + 1];
  if (r1 <= r0) return;             // nothing routed to this expert (block-uniform)
  if (warp == 0) {
    if (lane == 0) {
      mbar_init(&bar, 1);
      fence_mbar_init();
      mbar_arrive_expect_tx(&bar, uint32_t(ROWS) * (wt.wbytes() + 2 * wt.sbytes()));
    }
    __syncwarp();
    for (int r = lane; r < ROWS; r += 32) {
      size_t grow;
      if (SWIGLU) {
        const int tl = r >> 4, rr = r & 15;
        const int i = min(first + tl * 8 + (rr & 7), N - 1);
        grow = size_t(e) * 2 * N + (rr < 8 ? i : N + i);
      } else {
        grow = size_t(e) * N + min(first + r, N - 1);
      }
      wt.issue_row(wimg, ROWS, r, w, scales, biases, grow, &bar);
    }
  }
  int G0, G1;
  warp_group_range(K >> 6, warp, G0, G1);
  for (int c0 = r0; c0 < r1; c0 += NCOLS) {
    const int nc = min(NCOLS, r1 - c0);
    // columns beyond nc keep whatever they held: MMA columns are independent and theirs are not stored
#pragma unroll
    for (int b = 0; b < NCOLS; ++b)
      if (b < nc) QStage::stage(xst + b * cstride, x + size_t(c0 + b) * x_stride, nullptr, K, nullptr);
    __syncthreads();
    if (c0 == r0) wait_weights(&bar, 0);
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      qmv_tile_groups<NCOLS>(wt, wimg, ROWS, tl * 16 + g, tl * 16 + g + 8, xst, cstride, G0, G1, acc);
      part[warp][tl][g][2 * t] = acc[0]; part[warp][tl][g][2 * t + 1] = acc[1];
      part[warp][tl][g + 8][2 * t] = acc[2]; part[warp][tl][g + 8][2 * t + 1] = acc[3];
    }
    __syncthreads();
    if (SWIGLU) {
      for (int idx = threadIdx.x; idx < TILES * 8 * NCOLS; idx += kQThreads) {
        const int col = idx / (TILES * 8), rem = idx - col * (TILES * 8);
        const int tl = rem >> 3, gg = rem & 7, i = first + tl * 8 + gg;
        if (col >= nc || i >= N) continue;
        float gt = 0.f, up = 0.f;
#pragma unroll
        for (int wv = 0; wv < kQWarps; ++wv) { gt += part[wv][tl][gg][col]; up += part[wv][tl][gg + 8][col]; }
        out[size_t(c0 + col) * out_stride + i] = __float2bfloat16_rn(gt / (1.f + __expf(-gt)) * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < ROWS * NCOLS; idx += kQThreads) {
        const int col = idx / ROWS, rr = idx - col * ROWS, n = first + rr;
        if (col >= nc || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < kQWarps; ++wv) v += part[wv][rr >> 4][rr & 15][col];
        out[size_t(c0 + col) * out_stride + n] = __float2bfloat16_rn(v);
      }
    }
    __syncthreads();                // the next chunk overwrites the staged columns and the partials
  }
  pdl_launch_dependents();
}

}  // namespace rb

using namespace rb;

extern "C" int rmlx_qmv_mma_max_batch() { return 8; }

// 0 while every bulk-copy wait completed; kStatusMbarTimeout otherwise. Reading resets it.
extern "C" int rmlx_qmv_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_qmv_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_qmv_status, &zero, sizeof(int));
  return v;
}

// 1 when the shape can take this path.
extern "C" int rmlx_qmv_mma_supported(int K, int cols, int rows_per_block) {
  if (K % 512) return 0;
  const WTile wt{K};
  const size_t smem = ((wt.bytes(rows_per_block) + 127) & ~size_t(127)) + QStage::col_bytes(K) * cols;
  return smem <= 200 * 1024;
}

template <int NCOLS, int TILES, bool F32>
static int launch_rms_qmv(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                          const void* norm_w, float eps, const void* res, int res_stride, void* out,
                          int out_stride, int N, int K, int pdl, cudaStream_t st) {
  const WTile wt{K};
  const size_t smem = ((wt.bytes(16 * TILES) + 127) & ~size_t(127)) + QStage::col_bytes(K) * NCOLS;
  auto kern = rms_qmv_mma_kernel<NCOLS, TILES, F32>;
  RB_CHECK(set_max_smem(kern, smem));
  const int grid = (N + 16 * TILES - 1) / (16 * TILES);
  return launch(kern, dim3(grid), dim3(kQThreads), smem, st, pdl != 0,
                static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(sc),
                static_cast<const __nv_bfloat16*>(bi), static_cast<const __nv_bfloat16*>(x), x_stride,
                static_cast<const __nv_bfloat16*>(norm_w), eps,
                static_cast<const __nv_bfloat16*>(res), res_stride, out, out_stride, N, K);
}

// Q4 weights only (w uint32 [N, K/8], scales/biases bf16 [N, K/64]); K a multiple of 512;
// 1 <= B <= 8 activation rows.
extern "C" int rmlx_rms_qmv_mma(const void* w, const void* scales, const void* biases, const void* x,
                                int x_stride, const void* norm_w, float eps, const void* residual,
                                int res_stride, void* out, int out_stride, int out_f32, int B, int N,
                                int K, int pdl, cudaStream_t st) {
  if (B < 1 || B > 8 || N < 1) return -2;
  const bool big = N > 16384 && rmlx_qmv_mma_supported(K, B, 32);
  if (!rmlx_qmv_mma_supported(K, B, big ? 32 : 16)) return -2;
#define RB_QMV(NC)                                                                                   \
  case NC:                                                                                           \
    if (big) return out_f32 ? launch_rms_qmv<NC, 2, true>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st) \
                            : launch_rms_qmv<NC, 2, false>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st); \
    return out_f32 ? launch_rms_qmv<NC, 1, true>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st) \
                   : launch_rms_qmv<NC, 1, false>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st);
  switch (B) {
    RB_QMV(1) RB_QMV(2) RB_QMV(3) RB_QMV(4) RB_QMV(5) RB_QMV(6) RB_QMV(7) RB_QMV(8)
  }
#undef RB_QMV
  return -2;
}

extern "C" int rmlx_moe_gate_up_q4_mma(const void* w, const void* scales, const void* biases,
                                       const void* x, int x_stride, const void* norm_w, float eps,
                                       const int* topk_idx, void* act, int act_stride, int B,
                                       int top_k, int I, int K, int expert_base, int experts_local,
                                       int pdl, cudaStream_t st) {
  constexpr int TILES = 2;
  if (B < 1 || top_k < 1 || top_k > kQMaxTopK || I < 1) return -2;
  if (!rmlx_qmv_mma_supported(K, 1, 16 * TILES)) return -2;
  const WTile wt{K};
  const size_t smem = ((wt.bytes(16 * TILES) + 127) & ~size_t(127)) + QStage::col_bytes(K);
  auto kern = moe_gate_up_q4_mma_kernel<TILES>;
  RB_CHECK(set_max_smem(kern, smem));
  const int gx = (I + 8 * TILES - 1) / (8 * TILES);
  return launch(kern, dim3(gx, B * top_k), dim3(kQThreads), smem, st, pdl != 0,
                static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(scales),
                static_cast<const __nv_bfloat16*>(biases), static_cast<const __nv_bfloat16*>(x),
                x_stride, static_cast<const __nv_bfloat16*>(norm_w), eps, topk_idx,
                static_cast<__nv_bfloat16*>(act), act_stride, I, K, top_k, expert_base,
                experts_local);
}

extern "C" int rmlx_moe_down_q4_mma_supported(int I, int top_k) {
  if (I % 512 || top_k < 1 || top_k > kQMaxTopK) return 0;
  const WTile wt{I};
  const size_t smem = (((wt.bytes(16) + 127) & ~size_t(127)) + QStage::col_bytes(I)) * top_k;
  return smem <= 200 * 1024;
}

extern "C" int rmlx_moe_down_q4_mma(const void* w, const void* scales, const void* biases,
                                    const void* act, int act_stride, const int* topk_idx,
                                    const float* topk_w, const void* residual, int res_stride,
                                    void* out, int out_stride, int out_f32, int B, int top_k, int N,
                                    int I, int expert_base, int experts_local, int pdl,
                                    cudaStream_t st) {
  if (B < 1 || N < 1 || !rmlx_moe_down_q4_mma_supported(I, top_k)) return -2;
  const WTile wt{I};
  const size_t smem = (((wt.bytes(16) + 127) & ~size_t(127)) + QStage::col_bytes(I)) * top_k;
  const int gx = (N + 15) / 16;
#define RB_QDOWN(F32)                                                                              \
  {                                                                                                \
    auto kern = moe_down_q4_mma_kernel<F32>;                                                       \
    RB_CHECK(set_max_smem(kern, smem));                                                            \
    return launch(kern, dim3(gx, B), dim3(kQThreads), smem, st, pdl != 0,                          \
                  static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(scales),      \
                  static_cast<const __nv_bfloat16*>(biases), static_cast<const __nv_bfloat16*>(act), \
                  act_stride, topk_idx, topk_w, static_cast<const __nv_bfloat16*>(residual),       \
                  res_stride, out, out_stride, N, I, top_k, expert_base, experts_local);           \
  }
  if (out_f32) RB_QDOWN(true) else RB_QDOWN(false)
#undef RB_QDOWN
}

// Shapes the grouped narrow-M kernels take: K a multiple of 512 and the block's image within
// shared memory for the chosen variant (0: 8 columns x 16 rows; 1: 4 columns x 32 rows).
extern "C" int rmlx_moe_grouped_q4_mma_supported(int K, int variant) {
  if (K % 512 || variant < 0 || variant > 1) return 0;
  const WTile wt{K};
  const size_t smem = ((wt.bytes(variant ? 32 : 16) + 127) & ~size_t(127)) + QStage::col_bytes(K) * (variant ? 4 : 8);
  return smem <= 200 * 1024;
}

template <int NCOLS, int TILES, bool SWIGLU>
static int launch_grouped_qmv(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                              const int* offsets, void* out, int out_stride, int experts, int N, int K,
                              int pdl, cudaStream_t st) {
  const WTile wt{K};
  const size_t smem = ((wt.bytes(16 * TILES) + 127) & ~size_t(127)) + QStage::col_bytes(K) * NCOLS;
  auto kern = grouped_qmv_mma_kernel<NCOLS, TILES, SWIGLU>;
  RB_CHECK(set_max_smem(kern, smem));
  const int per = SWIGLU ? 8 * TILES : 16 * TILES;
  return launch(kern, dim3((N + per - 1) / per, experts), dim3(kQThreads), smem, st, pdl != 0,
                static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(sc),
                static_cast<const __nv_bfloat16*>(bi), static_cast<const __nv_bfloat16*>(x), x_stride,
                offsets, static_cast<__nv_bfloat16*>(out), out_stride, N, K);
}

// x [R, K] bf16, rows grouped by expert: rows offsets[e] .. offsets[e+1] belong to local expert e
// (offsets: experts + 1 ints on the device, absolute row numbers). swiglu != 0: w [experts, 2 N, K]
// -> out[r, 0..N) = silu(gate) * up; else w [experts, N, K] -> out[r, 0..N). Rows of x outside
// every local expert's range leave their rows of out untouched.
extern "C" int rmlx_moe_grouped_q4_mma(const void* w, const void* scales, const void* biases,
                                       const void* x, int x_stride, const int* offsets, void* out,
                                       int out_stride, int experts, int N, int K, int swiglu,
                                       int variant, int pdl, cudaStream_t st) {
  if (experts < 1 || experts > 65535 || N < 1 || !rmlx_moe_grouped_q4_mma_supported(K, variant)) return -2;
#define RB_GQ(NC, TL)                                                                               \
  return swiglu ? launch_grouped_qmv<NC, TL, true>(w, scales, biases, x, x_stride, offsets, out, out_stride, experts, N, K, pdl, st) \
                : launch_grouped_qmv<NC, TL, false>(w, scales, biases, x, x_stride, offsets, out, out_stride, experts, N, K, pdl, st);
  if (variant == 0) { RB_GQ(8, 1) }
  RB_GQ(4, 2)
#undef RB_GQ
}
