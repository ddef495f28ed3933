// Decode-time attention input in ONE kernel: RMSNorm + merged QKV projection + RoPE on Q and K +
// append of K and V to their page slots. A warp owns the two output rows that RoPE rotates together
// (i and i + HD/2 of one head, or 2i and 2i+1 in the traditional layout), so the rotation happens in
// registers on the fp32 dot products and the projection's output never goes to memory un-rotated.
// Positions, block tables and the row->sequence map are device buffers (shape-stable under CUDA
// graph replay).
//
// Fuses what the reference runs as three dispatches: rms_norm+gemv, rope_qk(v)_batch and
// kv_cache_copy_batched (crates/rmlx-core/src/ops/fused.rs:1530, crates/rmlx-core/src/ops/rope.rs:
// 500-870, crates/rmlx-core/src/ops/copy.rs:554).
#include "../common/gemv_core.cuh"
#include "../common/launch.cuh"

namespace rb {

template <class WT>
struct QkvMatrix;
template <>
struct QkvMatrix<WBf16> {
  using Row = RowBf16;
  const __nv_bfloat16* w; int K;
  __device__ Row row(size_t n) const { return Row{w + n * size_t(K)}; }
};
template <>
struct QkvMatrix<WQ4> {
  using Row = RowQ4;
  const uint32_t* w; const __nv_bfloat16* s; const __nv_bfloat16* b; int K;
  __device__ Row row(size_t n) const {
    return Row{w + n * size_t(K >> 3), s + n * size_t(K >> 6), b + n * size_t(K >> 6)};
  }
};

struct QkvRopeArgs {
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

template <class WT, int B>
__global__ void __launch_bounds__(kGemvThreads)
rms_qkv_rope_kernel(QkvMatrix<WT> W, const __nv_bfloat16* __restrict__ x, int x_stride,
                    const __nv_bfloat16* __restrict__ norm_w, float eps, QkvRopeArgs a) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float red[kGemvWarps];
  __shared__ float inv_rms[B];
  const int K = W.K, half = a.HD >> 1;
  const int pairs = (a.Hq + 2 * a.Hkv) * half;
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename QkvMatrix<WT>::Row;

  auto pair_rows = [&](int p, int& lo, int& hi) {
    const int head = p / half, i = p % half;
    lo = head * a.HD + (a.traditional ? 2 * i : i);
    hi = head * a.HD + (a.traditional ? 2 * i + 1 : i + half);
  };
  int p = blockIdx.x * kGemvWarps + warp;
  Row rows[2];
  Tile<Row, 2> t0;
  if (p < pairs) {       // the first tile of both rows flies during the wait and the staging
    int lo, hi;
    pair_rows(p, lo, hi);
    rows[0] = W.row(lo); rows[1] = W.row(hi);
    load_tile<2>(rows, K, 0, t0);
  }
  pdl_launch_dependents();
  pdl_wait();
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const float ssq = XStage<WT>::stage(smem + b * bstride, x + size_t(b) * x_stride, norm_w, K, red,
                                        norm_w != nullptr);
    if (threadIdx.x == 0) inv_rms[b] = norm_w ? rsqrtf(ssq / float(K) + eps) : 1.f;
  }
  __syncthreads();

  for (bool first = true; p < pairs; p += gridDim.x * kGemvWarps, first = false) {
    int lo, hi;
    pair_rows(p, lo, hi);
    if (!first) {
      rows[0] = W.row(lo); rows[1] = W.row(hi);
      load_tile<2>(rows, K, 0, t0);
    }
    float acc[2][B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[0][b] = acc[1][b] = 0.f;
    warp_dot<2, B, Row>(rows, smem, bstride, K, acc, t0);
    float mylo = 0.f, myhi = 0.f;           // lane b keeps batch row b's pair
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float s0 = warp_sum(acc[0][b]), s1 = warp_sum(acc[1][b]);
      if (lane == b) { mylo = s0 * inv_rms[b]; myhi = s1 * inv_rms[b]; }
    }
    if (lane < B) {
      const int b = lane, head = p / half, i = p % half;
      const int pos = a.positions[b];
      const int d_lo = lo - head * a.HD, d_hi = hi - head * a.HD;
      if (head < a.Hq + a.Hkv) {             // rotate Q and K
        const float c = a.cos_t[size_t(pos) * half + i], s = a.sin_t[size_t(pos) * half + i];
        const float r0 = mylo * c - myhi * s, r1 = myhi * c + mylo * s;
        mylo = r0; myhi = r1;
      }
      __nv_bfloat16* dst;
      if (head < a.Hq) {
        dst = a.q_out + (size_t(b) * a.Hq + head) * a.HD;
      } else {
        const int seq = a.row_seq ? a.row_seq[b] : b;
        const bool inb = RB_BOUNDS(pos / a.page, a.max_blocks);   // bounds-checked build: skip the append
        const int blk = inb ? a.block_table[size_t(seq) * a.max_blocks + pos / a.page] : 0;
        const bool is_k = head < a.Hq + a.Hkv;
        const int kvh = is_k ? head - a.Hq : head - a.Hq - a.Hkv;
        dst = inb ? (is_k ? a.k_cache : a.v_cache) + ((size_t(blk) * a.Hkv + kvh) * a.page + pos % a.page) * a.HD
                  : nullptr;
      }
      if (dst) {
        dst[d_lo] = __float2bfloat16_rn(mylo);
        dst[d_hi] = __float2bfloat16_rn(myhi);
      }
    }
  }
  pdl_launch_dependents();
}

template <class WT>
static QkvMatrix<WT> make_qkv(const void* w, const void* s, const void* b, int K);
template <>
QkvMatrix<WBf16> make_qkv<WBf16>(const void* w, const void*, const void*, int K) {
  return QkvMatrix<WBf16>{static_cast<const __nv_bfloat16*>(w), K};
}
template <>
QkvMatrix<WQ4> make_qkv<WQ4>(const void* w, const void* s, const void* b, int K) {
  return QkvMatrix<WQ4>{static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(s),
                        static_cast<const __nv_bfloat16*>(b), K};
}

template <class WT, int B>
static int launch_qkv_rope(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                           const void* norm_w, float eps, const QkvRopeArgs& a, int K, int pdl,
                           cudaStream_t st) {
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const size_t smem = bstride * B;
  auto kern = rms_qkv_rope_kernel<WT, B>;
  RB_CHECK(set_max_smem(kern, smem));
  const int pairs = (a.Hq + 2 * a.Hkv) * (a.HD / 2);
  const int want = (pairs + kGemvWarps - 1) / kGemvWarps, cap = sm_count() * 8;
  return launch(kern, dim3(want < cap ? want : cap), dim3(kGemvThreads), smem, st, pdl != 0,
                make_qkv<WT>(w, sc, bi, K), static_cast<const __nv_bfloat16*>(x), x_stride,
                static_cast<const __nv_bfloat16*>(norm_w), eps, a);
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("decode_qkv_rope.cu")


// x [B, K] bf16 -> Q rotated into q_out [B, Hq, HD]; K rotated and V copied into their page slots.
// w: merged QKV weight [(Hq + 2*Hkv) * HD, K] (w_kind 0 bf16, 1 MLX-affine Q4). B <= 4.
extern "C" int rmlx_rms_qkv_rope(int w_kind, const void* w, const void* scales, const void* biases,
                                 const void* x, int x_stride, const void* norm_w, float eps,
                                 void* q_out, void* k_cache, void* v_cache, const int* block_table,
                                 const int* positions, const int* row_seq, const float* cos_t,
                                 const float* sin_t, int B, int K, int Hq, int Hkv, int HD,
                                 int max_blocks, int page, int traditional, int pdl, cudaStream_t st) {
  if (K % 8 || (w_kind == 1 && K % 64) || B < 1 || B > 4 || HD % 2 || Hq < 1 || Hkv < 1) return -2;
  QkvRopeArgs a{static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
                static_cast<__nv_bfloat16*>(v_cache), block_table, positions, row_seq, cos_t, sin_t,
                Hq, Hkv, HD, max_blocks, page, traditional};
#define RB_QR(WT_)                                                                                       \
  switch (B) {                                                                                            \
    case 1: return launch_qkv_rope<WT_, 1>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st);   \
    case 2: return launch_qkv_rope<WT_, 2>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st);   \
    case 3: return launch_qkv_rope<WT_, 3>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st);   \
    default: return launch_qkv_rope<WT_, 4>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st);  \
  }
  if (w_kind == 0) { RB_QR(WBf16) }
  if (w_kind == 1) { RB_QR(WQ4) }
#undef RB_QR
  return -2;
}
