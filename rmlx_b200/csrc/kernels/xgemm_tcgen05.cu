// Generalised tcgen05 GEMM: C = A · W^T with
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
// warps 2-5 epilogue (TMEM -> registers -> bf16 global, + residual), warps 6-9 dequant (Q4 only).
// Accumulators are double-buffered in TMEM. All pipeline waits are bounded.
//
// Reference counterparts: affine_qmm_* (crates/rmlx-core/src/ops/quantized.rs:2871-6284; 17.43
// TFLOPS published for Q4 at M=512), grouped_gemm_mlx_f16 / gather_mm_*
// (crates/rmlx-core/src/ops/matmul.rs:5945, crates/rmlx-core/src/ops/gather_mm.rs:60-332).
#include <cuda.h>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.cuh"

namespace rb {

constexpr int kXBM = 128;
constexpr int kXBK = 64;
constexpr int kXMaxExperts = 256;

template <int BN, bool WQ4>
struct XSmem {
  static constexpr int kStages = WQ4 ? 3 : ((BN >= 256) ? 4 : 6);
  static constexpr int kRawStages = 4;
  static constexpr int kStageA = kXBM * kXBK * 2;
  static constexpr int kStageB = BN * kXBK * 2;
  static constexpr int kStageRaw = BN * 32;          // 64 nibbles per row
  static constexpr int kScaleSlot = 2 * BN * 16;     // scales + biases for 8 k-blocks
  static constexpr int kBytes = kStages * (kStageA + kStageB) +
                                (WQ4 ? kRawStages * kStageRaw + 2 * kScaleSlot : 0) + 1024 + 512 +
                                (kXMaxExperts + 2) * 8;
  static constexpr int kThreads = WQ4 ? 320 : 192;
};

struct XTile {
  int a_row0;     // first row of the A/C tile
  int row_end;    // rows >= row_end are not stored
  int w_row0;     // first row of the W tile (in the stacked weight)
  int c_col0;     // first output column
};

// tile id -> coordinates. Plain: column-block major so consecutive CTAs share a W tile.
template <int BN, bool GROUPED>
__device__ __forceinline__ XTile x_tile(int tile, int M, int N, int tiles_m, int tiles_n,
                                        const int* s_off, const int* s_tprefix, int E) {
  XTile t;
  if (!GROUPED) {
    const int tm = tile % tiles_m, tn = tile / tiles_m;
    t.a_row0 = tm * kXBM; t.row_end = M; t.w_row0 = tn * BN; t.c_col0 = tn * BN;
  } else {
    int e = 0;
    while (e + 1 < E && s_tprefix[e + 1] <= tile) ++e;
    while (s_tprefix[e + 1] <= tile) ++e;                 // skips empty experts
    const int local = tile - s_tprefix[e];
    const int rows = s_off[e + 1] - s_off[e];
    const int mt_e = (rows + kXBM - 1) / kXBM;
    const int nt = local / mt_e, mt = local % mt_e;
    t.a_row0 = s_off[e] + mt * kXBM; t.row_end = s_off[e + 1];
    t.w_row0 = e * N + nt * BN; t.c_col0 = nt * BN;
  }
  return t;
}

template <int BN, bool WQ4, bool GROUPED, bool RESIDUAL>
__global__ void __launch_bounds__((XSmem<BN, WQ4>::kThreads), 1)
xgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
             const __grid_constant__ CUtensorMap tmap_s, const __grid_constant__ CUtensorMap tmap_b,
             __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ residual,
             const int* __restrict__ offsets, int E, int M, int N, int K, int ldc,
             int* __restrict__ status) {
  using S = XSmem<BN, WQ4>;
  constexpr int STAGES = S::kStages, RAW = S::kRawStages;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : 2 * BN;
  extern __shared__ char smem_raw[];
  char* smem = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  char* sA = smem;
  char* sB = sA + STAGES * S::kStageA;
  char* sRaw = sB + STAGES * S::kStageB;
  char* sScale = sRaw + (WQ4 ? RAW * S::kStageRaw : 0);
  char* after = sScale + (WQ4 ? 2 * S::kScaleSlot : 0);
  uint64_t* bars = reinterpret_cast<uint64_t*>(after);
  uint64_t* full = bars;                        // [STAGES] A (and bf16 B) landed
  uint64_t* empty = full + STAGES;              // [STAGES] MMAs finished reading the stage
  uint64_t* bq_full = empty + STAGES;           // [STAGES] dequantised B written (Q4)
  uint64_t* raw_full = bq_full + STAGES;        // [RAW]
  uint64_t* raw_empty = raw_full + RAW;         // [RAW]
  uint64_t* sc_full = raw_empty + RAW;          // [2]
  uint64_t* sc_empty = sc_full + 2;             // [2]
  uint64_t* acc_full = sc_empty + 2;            // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* s_off = reinterpret_cast<int*>(after + 512);          // [E+1]
  int* s_tprefix = s_off + kXMaxExperts + 1;                 // [E+1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN;
  int tiles_m = (M + kXBM - 1) / kXBM;
  const int num_kb = (K + kXBK - 1) / kXBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); mbar_init(bq_full + i, 4); }
    for (int i = 0; i < RAW; ++i) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, 4); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(sc_full + i, 1); mbar_init(sc_empty + i, 4);
      mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 4);
    }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (GROUPED) {
    pdl_wait();
    for (int i = threadIdx.x; i <= E; i += blockDim.x) s_off[i] = offsets[i];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (GROUPED) {
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int e = 0; e < E; ++e) {
        s_tprefix[e] = acc;
        acc += ((s_off[e + 1] - s_off[e] + kXBM - 1) / kXBM) * tiles_n;
      }
      s_tprefix[E] = acc;
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? s_tprefix[E] : tiles_m * tiles_n;
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      if (!GROUPED) pdl_wait();
      int stage = 0, rstage = 0, sslot = 0;
      uint32_t phase = 0, rphase = 0, sphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const XTile t = x_tile<BN, GROUPED>(tile, M, N, tiles_m, tiles_n, s_off, s_tprefix, E);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (WQ4) {
            if ((kb & 7) == 0) {
              if (!mbar_wait(sc_empty + sslot, sphase ^ 1u, abort_flag)) { ok = false; break; }
              mbar_arrive_expect_tx(sc_full + sslot, S::kScaleSlot);
              tma_load_2d(sScale + sslot * S::kScaleSlot, &tmap_s, sc_full + sslot, kb, t.w_row0);
              tma_load_2d(sScale + sslot * S::kScaleSlot + BN * 16, &tmap_b, sc_full + sslot, kb, t.w_row0);
              if (++sslot == 2) { sslot = 0; sphase ^= 1u; }
            }
            if (!mbar_wait(raw_empty + rstage, rphase ^ 1u, abort_flag)) { ok = false; break; }
            mbar_arrive_expect_tx(raw_full + rstage, S::kStageRaw);
            tma_load_2d(sRaw + rstage * S::kStageRaw, &tmap_w, raw_full + rstage, kb * 32, t.w_row0);
            if (++rstage == RAW) { rstage = 0; rphase ^= 1u; }
          }
          if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          mbar_arrive_expect_tx(full + stage, S::kStageA + (WQ4 ? 0 : S::kStageB));
          tma_load_2d(sA + stage * S::kStageA, &tmap_a, full + stage, kb * kXBK, t.a_row0);
          if (!WQ4) tma_load_2d(sB + stage * S::kStageB, &tmap_w, full + stage, kb * kXBK, t.w_row0);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kXBM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(acc_empty + acc, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase, abort_flag)) { ok = false; break; }
          if (WQ4 && !mbar_wait(bq_full + stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kStageA);
          const uint32_t b_addr = smem_u32(sB + stage * S::kStageB);
#pragma unroll
          for (int k = 0; k < kXBK / 16; ++k)
            tc_mma_f16(d_tmem, umma_desc_sw128_kmajor(a_addr + k * 32),
                       umma_desc_sw128_kmajor(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(empty + stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(acc_full + acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    if (RESIDUAL && !GROUPED) pdl_wait();
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const XTile t = x_tile<BN, GROUPED>(tile, M, N, tiles_m, tiles_n, s_off, s_tprefix, E);
      if (!mbar_wait(acc_full + acc, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = t.a_row0 + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = t.c_col0 + c * 32;
        if (row < t.row_end && col0 < N) {
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
  } else if (WQ4) {
    // ------------------------------------------------------------------ dequant (warps 6..9)
    const int dt = threadIdx.x - 192;   // 0..127
    int stage = 0, rstage = 0, sslot = 0;
    uint32_t phase = 0, rphase = 0, sphase = 0;
    bool ok = true;
    const __nv_bfloat162 k128 = __float2bfloat162_rn(128.f);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb) {
        if ((kb & 7) == 0 && !mbar_wait(sc_full + sslot, sphase, abort_flag)) { ok = false; break; }
        if (!mbar_wait(raw_full + rstage, rphase, abort_flag)) { ok = false; break; }
        if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag)) { ok = false; break; }  // B slot free
        const char* raw = sRaw + rstage * S::kStageRaw;
        const __nv_bfloat16* sc = reinterpret_cast<const __nv_bfloat16*>(sScale + sslot * S::kScaleSlot);
        const __nv_bfloat16* bi = sc + BN * 8;
        char* bst = sB + stage * S::kStageB;
#pragma unroll
        for (int it = 0; it < (BN * 2) / 128; ++it) {
          const int item = it * 128 + dt;
          const int r = item % BN, h = item / BN;     // row of the W tile, which half of the 64 k
          const uint4 wv = *reinterpret_cast<const uint4*>(raw + r * 32 + h * 16);
          const __nv_bfloat162 s2 = __bfloat162bfloat162(sc[r * 8 + (kb & 7)]);
          const __nv_bfloat162 b2 = __bfloat162bfloat162(bi[r * 8 + (kb & 7)]);
          const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t w = words[j];
            // (128 + q) is exact in bf16: the nibble goes into the low mantissa bits of 128.0
            uint32_t p04 = (w & 0x000f000fu) | 0x43004300u;            // (k0, k4)
            uint32_t p15 = ((w >> 4) & 0x000f000fu) | 0x43004300u;     // (k1, k5)
            uint32_t p26 = ((w >> 8) & 0x000f000fu) | 0x43004300u;     // (k2, k6)
            uint32_t p37 = ((w >> 12) & 0x000f000fu) | 0x43004300u;    // (k3, k7)
            __nv_bfloat162 v04 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p04), k128), s2, b2);
            __nv_bfloat162 v15 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p15), k128), s2, b2);
            __nv_bfloat162 v26 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p26), k128), s2, b2);
            __nv_bfloat162 v37 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p37), k128), s2, b2);
            const uint32_t u04 = *reinterpret_cast<uint32_t*>(&v04), u15 = *reinterpret_cast<uint32_t*>(&v15);
            const uint32_t u26 = *reinterpret_cast<uint32_t*>(&v26), u37 = *reinterpret_cast<uint32_t*>(&v37);
            uint4 o;   // natural k order: (k0,k1) (k2,k3) (k4,k5) (k6,k7)
            o.x = __byte_perm(u04, u15, 0x5410); o.y = __byte_perm(u26, u37, 0x5410);
            o.z = __byte_perm(u04, u15, 0x7632); o.w = __byte_perm(u26, u37, 0x7632);
            const int c = h * 4 + j;                   // 16-byte chunk of the 128-byte row
            *reinterpret_cast<uint4*>(bst + r * 128 + ((c ^ (r & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_smem();     // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bq_full + stage);
          mbar_arrive(raw_empty + rstage);
          if ((kb & 7) == 7 || kb == num_kb - 1) mbar_arrive(sc_empty + sslot);
        }
        if ((kb & 7) == 7 || kb == num_kb - 1) { if (++sslot == 2) { sslot = 0; sphase ^= 1u; } }
        if (++rstage == RAW) { rstage = 0; rphase ^= 1u; }
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, kStatusMbarTimeout);
  pdl_launch_dependents();
}

template <int BN, bool WQ4, bool GROUPED, bool RESIDUAL>
static int launch_x(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& ts,
                    const CUtensorMap& tb, void* C, const void* residual, const int* offsets, int E,
                    int M, int N, int K, int ldc, int* status, int pdl, cudaStream_t st) {
  using S = XSmem<BN, WQ4>;
  auto kern = xgemm_kernel<BN, WQ4, GROUPED, RESIDUAL>;
  RB_CHECK(set_max_smem(kern, S::kBytes));
  int tiles = ((M + kXBM - 1) / kXBM) * ((N + BN - 1) / BN);
  if (GROUPED) tiles += E * ((N + BN - 1) / BN);   // upper bound: every group may add a ragged tile
  const int grid = tiles < sm_count() ? (tiles > 0 ? tiles : 1) : sm_count();
  return launch(kern, dim3(grid), dim3(S::kThreads), size_t(S::kBytes), st, pdl != 0, ta, tw, ts, tb,
                static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(residual), offsets, E,
                M, N, K, ldc, status);
}

}  // namespace rb

using namespace rb;

// 1 when the Q4 fast path can take this K (TMA needs 16-byte row strides for the scale arrays).
extern "C" int rmlx_qgemm_supported(int K) { return K % 512 == 0; }

// C[M,N] = A[M,K] * W^T (+ residual), bf16 out.
//   w_kind 0: W bf16 [rowsW, K];  w_kind 1: packed uint32 [rowsW, K/8] + scales/biases bf16 [rowsW, K/64]
//   offsets == nullptr: plain GEMM, rowsW = N.
//   offsets != nullptr: grouped; A rows are sorted by expert, offsets[E+1] (device, int32),
//                       rowsW = E*N, N must be a multiple of the tile width.
extern "C" int rmlx_xgemm(int w_kind, const void* A, const void* W, const void* scales,
                          const void* biases, void* C, const void* residual, const int* offsets,
                          int E, int M, int N, int K, int lda, int ldc, int bn, int* status, int pdl,
                          cudaStream_t st) {
  if (M < 1 || N < 1 || K < 8 || K % 8 || lda % 8) return -2;
  if (w_kind == 1 && !rmlx_qgemm_supported(K)) return -2;
  const bool grouped = offsets != nullptr;
  if (grouped && (E < 1 || E > kXMaxExperts)) return -2;
  if (bn == 0) bn = (grouped || w_kind == 1) ? ((N % 256 == 0 && M >= 1024) ? 256 : 128) : 128;
  if (bn != 128 && bn != 256) return -2;
  if (grouped && N % bn) return -2;
  const uint64_t rowsW = grouped ? uint64_t(E) * N : uint64_t(N);
  CUtensorMap ta, tw, ts, tb;
  int rc = make_tmap_2d_bf16(&ta, A, uint64_t(K), uint64_t(M), uint64_t(lda) * 2, kXBK, kXBM);
  if (rc) return rc;
  if (w_kind == 0) {
    rc = make_tmap_2d_bf16(&tw, W, uint64_t(K), rowsW, uint64_t(K) * 2, kXBK, bn);
    if (rc) return rc;
    ts = tw; tb = tw;
  } else {
    rc = make_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, uint64_t(K) / 2, rowsW, uint64_t(K) / 2,
                      32, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tmap_2d(&ts, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, scales, uint64_t(K) / 64, rowsW,
                      uint64_t(K) / 64 * 2, 8, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, biases, uint64_t(K) / 64, rowsW,
                      uint64_t(K) / 64 * 2, 8, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
#define RB_X(BN_, Q_, G_)                                                                          \
  return residual ? launch_x<BN_, Q_, G_, true>(ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st) \
                  : launch_x<BN_, Q_, G_, false>(ta, tw, ts, tb, C, residual, offsets, E, M, N, K, ldc, status, pdl, st)
  if (bn == 256) {
    if (w_kind == 1) { if (grouped) { RB_X(256, true, true); } else { RB_X(256, true, false); } }
    else { if (grouped) { RB_X(256, false, true); } else { RB_X(256, false, false); } }
  } else {
    if (w_kind == 1) { if (grouped) { RB_X(128, true, true); } else { RB_X(128, true, false); } }
    else { if (grouped) { RB_X(128, false, true); } else { RB_X(128, false, false); } }
  }
#undef RB_X
}
