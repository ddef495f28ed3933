// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] · W[N,K]^T (+ residual), fp32
// accumulation in tensor memory.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128x64 A tiles and BNx64 W tiles (128-byte swizzle) into a ring of
//               shared-memory stages, completion on mbarriers
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times
//               per stage; tcgen05.commit releases the stage back to the producer and, at the end
//               of a tile, hands the accumulator to the epilogue
//   warps 2-5   epilogue: tcgen05.ld the 128xBN fp32 accumulator out of TMEM (each warp owns the
//               32 lanes its position in the warpgroup may touch), add the residual, convert to
//               bf16 and store
// Two accumulators (2 x BN columns of TMEM) let the epilogue of tile i overlap the main loop of
// tile i+1. Rows past M and columns past K are zero-filled by TMA; stores are predicated.
//
// Replaces the reference's simdgroup-MMA GEMM family and its tile-selection logic (gemm_mlx_*,
// gemm_nax_*, split-K; crates/rmlx-core/src/ops/matmul.rs:2160-5610,6377-6480) and the residual
// epilogue of matmul_add_residual_into_cb (matmul.rs:7988).
#include <cuda.h>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.cuh"

namespace rb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmSmem {
  static constexpr int kStageA = kBM * kBK * 2;
  static constexpr int kStageB = BN * kBK * 2;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kBytes = kStages * (kStageA + kStageB) + 1024 /*align slack*/ + 256 /*barriers*/;
};

// OUT_F32: the accumulator is stored as fp32 (C is then float*, ldc counts floats): router logits
// and other results that must not be rounded to bf16.
template <int BN, bool RESIDUAL, bool OUT_F32 = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_w,
                         void* __restrict__ Cv, const __nv_bfloat16* __restrict__ residual,
                         int M, int N, int K, int ldc, int* __restrict__ status) {
  __nv_bfloat16* C = static_cast<__nv_bfloat16*>(Cv);
  using S = GemmSmem<BN>;
  constexpr int STAGES = S::kStages;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : 2 * BN;  // power of two: BN in {32,..,256}
  extern __shared__ char smem_raw[];
  // tiles need 1024-byte alignment for the 128-byte swizzle
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* sA = smem;
  char* sB = smem + STAGES * S::kStageA;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + STAGES * S::kStageB);
  uint64_t* full = bars;                  // [STAGES]
  uint64_t* empty = bars + STAGES;        // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES; // [2]
  uint64_t* acc_empty = acc_full + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 4); }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 1) {  // this warp owns the TMEM allocation
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      pdl_wait();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        // consecutive CTAs share the same W tile column-block: good L2 reuse of W across M
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(full + stage, S::kStageA + S::kStageB);
          tma_load_2d(sA + stage * S::kStageA, &tmap_a, full + stage, kb * kBK, tm * kBM);
          tma_load_2d(sB + stage * S::kStageB, &tmap_w, full + stage, kb * kBK, tn * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(acc_empty + acc, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kStageA);
          const uint32_t b_addr = smem_u32(sB + stage * S::kStageB);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            tc_mma_f16(d_tmem, umma_desc_sw128_kmajor(a_addr + k * 32),
                       umma_desc_sw128_kmajor(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty + stage);  // stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(acc_full + acc);   // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    if (RESIDUAL) pdl_wait();
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      if (!mbar_wait(acc_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = tm * kBM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if (OUT_F32) {
          if (row < M && col0 < N) {
            float* dstf = static_cast<float*>(Cv) + size_t(row) * ldc + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) dstf[j] = __uint_as_float(r[j]);
          }
        } else if (row < M && col0 < N) {
          __nv_bfloat16* dst = C + size_t(row) * ldc + col0;
          const __nv_bfloat16* res = RESIDUAL ? residual + size_t(row) * ldc + col0 : nullptr;
          if (col0 + 32 <= N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              if (RESIDUAL) {
                const uint4 rv = *reinterpret_cast<const uint4*>(res + v * 8);
                f[0] += bf16lo(rv.x); f[1] += bf16hi(rv.x); f[2] += bf16lo(rv.y); f[3] += bf16hi(rv.y);
                f[4] += bf16lo(rv.z); f[5] += bf16hi(rv.z); f[6] += bf16lo(rv.w); f[7] += bf16hi(rv.w);
              }
              uint4 o;
              o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
              o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + v * 8) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < N) {
                float f = __uint_as_float(r[j]);
                if (RESIDUAL) f += __bfloat162float(res[j]);
                dst[j] = __float2bfloat16_rn(f);
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, kStatusMbarTimeout);
  pdl_launch_dependents();
}

template <int BN, bool RESIDUAL, bool OUT_F32 = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, void* C, const void* residual,
                       int M, int N, int K, int ldc, int* status, int pdl, cudaStream_t st) {
  auto kern = gemm_bf16_tcgen05_kernel<BN, RESIDUAL, OUT_F32>;
  constexpr size_t smem = GemmSmem<BN>::kBytes;
  RB_CHECK(set_max_smem(kern, smem));
  const int tiles = ((M + kBM - 1) / kBM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  return launch(kern, dim3(grid), dim3(kGemmThreads), smem, st, pdl != 0, ta, tw, C,
                static_cast<const __nv_bfloat16*>(residual), M, N, K, ldc, status);
}

}  // namespace rb

using namespace rb;

// Tile width heuristic: the widest N tile that still yields about one tile per SM.
extern "C" int rmlx_gemm_pick_bn(int M, int N) {
  const int tm = (M + kBM - 1) / kBM;
  const int sms = sm_count();
  const int cands[4] = {256, 128, 64, 32};
  for (int i = 0; i < 4; ++i) {
    const int bn = cands[i];
    if (tm * ((N + bn - 1) / bn) >= sms || bn == 32) return bn;
  }
  return 32;
}

// C[M,N] (bf16, row stride ldc) = A[M,K] (bf16, row stride lda) * W[N,K]^T (bf16, row stride ldw)
// (+ residual[M,N] with C's stride). K, lda, ldw multiples of 8; A and W 16-byte aligned.
// bn: 0 = choose, else one of 32/64/128/256. status: optional device int set non-zero if a
// pipeline wait gave up.
extern "C" int rmlx_gemm_bf16(const void* A, const void* W, void* C, const void* residual, int M,
                              int N, int K, int lda, int ldw, int ldc, int bn, int* status, int pdl,
                              cudaStream_t st) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldw % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -2;
  if (bn == 0) bn = rmlx_gemm_pick_bn(M, N);
  CUtensorMap ta, tw;
  int rc = make_tmap_2d_bf16(&ta, A, uint64_t(K), uint64_t(M), uint64_t(lda) * 2, kBK, kBM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tw, W, uint64_t(K), uint64_t(N), uint64_t(ldw) * 2, kBK, bn);
  if (rc) return rc;
#define RB_GEMM(BN_)                                                                              \
  case BN_:                                                                                       \
    return residual ? launch_gemm<BN_, true>(ta, tw, C, residual, M, N, K, ldc, status, pdl, st)  \
                    : launch_gemm<BN_, false>(ta, tw, C, residual, M, N, K, ldc, status, pdl, st);
  switch (bn) {
    RB_GEMM(256)
    RB_GEMM(128)
    RB_GEMM(64)
    RB_GEMM(32)
    default: return -2;
  }
#undef RB_GEMM
}

// The same product with an fp32 result: C[M,N] float, row stride ldc floats. No residual.
extern "C" int rmlx_gemm_bf16_f32(const void* A, const void* W, void* C, int M, int N, int K, int lda,
                                  int ldw, int ldc, int* status, int pdl, cudaStream_t st) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8 || ldw % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -2;
  const int bn = rmlx_gemm_pick_bn(M, N) >= 128 ? 128 : 64;
  CUtensorMap ta, tw;
  int rc = make_tmap_2d_bf16(&ta, A, uint64_t(K), uint64_t(M), uint64_t(lda) * 2, kBK, kBM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tw, W, uint64_t(K), uint64_t(N), uint64_t(ldw) * 2, kBK, bn);
  if (rc) return rc;
  if (bn == 128) return launch_gemm<128, false, true>(ta, tw, C, nullptr, M, N, K, ldc, status, pdl, st);
  return launch_gemm<64, false, true>(ta, tw, C, nullptr, M, N, K, ldc, status, pdl, st);
}
