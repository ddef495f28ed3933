// Generalised tcgen05 GEMM, single-GPU entry points: C = A · W^T with
//   * W either bf16 (TMA-fed) or MLX-affine Q4 (group 64) dequantised INSIDE the main loop:
//     packed nibbles and per-group scales/biases arrive by TMA, four dequant warps expand them to
//     bf16 (exactly s*q+b, rounded once) straight into the 128-byte-swizzled operand stage that
//     tcgen05.mma reads, so quantised weights never exist in memory in expanded form;
//   * an optional grouped mode for mixture-of-experts: rows of A are sorted by expert, a device
//     array of offsets [E+1] describes the groups, W is the stack [E*N, K]; every CTA derives the
//     tile table (expert, m-tile, n-tile) from the offsets itself, so empty experts cost nothing
//     and no host round trip is needed (the reference builds its tile table on the CPU,
//     crates/rmlx-core/src/ops/matmul.rs:8823-8950).
//
// Roles per CTA (persistent, one CTA per SM): warp 0 TMA producer, warp 1 MMA issuer (owns TMEM),
// warps 2-5 epilogue (TMEM -> registers -> bf16 global, + residual), warps 6-13 dequant (Q4 only).
// Accumulators are double-buffered in TMEM. All pipeline waits are bounded. The kernel itself is in
// xgemm_kernel.cuh.
//
// Reference counterparts: affine_qmm_* (crates/rmlx-core/src/ops/quantized.rs:2871-6284; 17.43
// TFLOPS published for Q4 at M=512), grouped_gemm_mlx_f16 / gather_mm_*
// (crates/rmlx-core/src/ops/matmul.rs:5945, crates/rmlx-core/src/ops/gather_mm.rs:60-332).
#include "xgemm_kernel.cuh"

using namespace rb;

// 1 when the Q4 fast path can take this K (TMA needs 16-byte row strides for the scale arrays).
extern "C" int rmlx_qgemm_supported(int K) { return K % 512 == 0; }

// C[M,N] = A[M,K] * W^T (+ residual), bf16 out.
//   w_kind 0: W bf16 [rowsW, K];  w_kind 1: packed uint32 [rowsW, K/8] + scales/biases bf16 [rowsW, K/64]
//   offsets == nullptr: plain GEMM, rowsW = N.
//   offsets != nullptr: grouped; A rows are sorted by expert, offsets[E+1] (device, int32),
//                       rowsW = E*N, N must be a multiple of the tile width.
//   swiglu != 0: W's N rows (per expert) are [gate; up]; C gets N/2 columns of silu(gate)*up,
//                computed in the epilogue from the fp32 accumulators (no residual in this mode).
extern "C" int rmlx_xgemm(int w_kind, const void* A, const void* W, const void* scales,
                          const void* biases, void* C, const void* residual, const int* offsets,
                          int E, int M, int N, int K, int lda, int ldc, int bn, int swiglu,
                          int* status, int pdl, cudaStream_t st) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8) return -2;
  if (w_kind == 1 && !rmlx_qgemm_supported(K)) return -2;
  const bool grouped = offsets != nullptr;
  if (grouped && (E < 1 || E > kXMaxExperts)) return -2;
  // bn < 0: stacked tiles (two 128-row blocks of A per staged block of W) of width |bn| = 128
  int mt = 1;
  if (bn < 0) { mt = 2; bn = -bn; }
  if (mt == 2 && (bn != 128 || (grouped && residual))) return -2;
  if (bn == 0) {
    bn = (grouped || w_kind == 1) ? ((N % 256 == 0 && M >= 1024) ? 256 : 128) : 128;
    // Q4, many rows: the dequant warps are the limit, so share each dequantised block of W
    // between two row blocks
    if (w_kind == 1 && !grouped && ((M + 255) / 256) * ((N + 127) / 128) >= 120) { bn = 128; mt = 2; }
    // grouped: experts with more than 128 rows share their dequantised blocks too (M is the total
    // row count; below ~256 rows per expert the wider single-block tile measures faster)
    if (w_kind == 1 && grouped && !residual && M >= 256 * E && N % 128 == 0) { bn = 128; mt = 2; }
    // few rows: the work is streaming W, so spread it over more SMs with narrower tiles
    if (!grouped && ((M + kXBM - 1) / kXBM) * ((N + 127) / 128) < 100) bn = 64;
  }
  if (bn != 64 && bn != 128 && bn != 256) return -2;
  if (grouped && N % bn) return -2;
  if (swiglu && (residual || N % bn)) return -2;
  const uint64_t rowsW = grouped ? uint64_t(E) * N : uint64_t(N);
  CUtensorMap ta, tw, ts, tb;
  int rc = make_tmap_2d_bf16(&ta, A, uint64_t(K), uint64_t(M), uint64_t(lda) * 2, kXBK, kXBM);
  if (rc) return rc;
  rc = x_weight_maps(w_kind, W, scales, biases, rowsW, K, swiglu ? bn / 2 : bn, &tw, &ts, &tb);
  if (rc) return rc;
#define RB_X(BN_, Q_, G_)                                                                          \
  return residual ? launch_x<BN_, Q_, G_, true>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st) \
                  : launch_x<BN_, Q_, G_, false>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st, XComm(), swiglu)
  if (mt == 2 && grouped) {
    if (w_kind == 1)
      return launch_x<128, true, true, false, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st, XComm(), swiglu);
    return launch_x<128, false, true, false, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st, XComm(), swiglu);
  }
  if (mt == 2) {
    if (w_kind == 1) {
      return residual ? launch_x<128, true, false, true, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st)
                      : launch_x<128, true, false, false, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st, XComm(), swiglu);
    }
    return residual ? launch_x<128, false, false, true, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st)
                    : launch_x<128, false, false, false, kCommNone, 2>(ta, ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st, XComm(), swiglu);
  }
  if (bn == 256) {
    if (w_kind == 1) { if (grouped) { RB_X(256, true, true); } else { RB_X(256, true, false); } }
    else { if (grouped) { RB_X(256, false, true); } else { RB_X(256, false, false); } }
  } else if (bn == 64) {
    if (w_kind == 1) { if (grouped) { RB_X(64, true, true); } else { RB_X(64, true, false); } }
    else { if (grouped) { RB_X(64, false, true); } else { RB_X(64, false, false); } }
  } else {
    if (w_kind == 1) { if (grouped) { RB_X(128, true, true); } else { RB_X(128, true, false); } }
    else { if (grouped) { RB_X(128, false, true); } else { RB_X(128, false, false); } }
  }
#undef RB_X
}
