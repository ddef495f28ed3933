// Paged causal flash attention for prompt processing on the 5th-generation tensor cores
// (head_dim 128, optional sliding window; other head dimensions use the mma.sync kernel in
// flash_prefill.cu).
//
// A CTA owns LANES (1 or 2) tiles of 128 query tokens of one query head and walks the keys 64 at a
// time; the K and V tiles of a step serve every lane. A kernel that allocates tensor memory gets one
// CTA per SM (the occupancy calculator reports 1 for any kernel with tcgen05.alloc), so a second
// lane is the only way to put two softmax warps on each scheduler: each lane has its own softmax
// warpgroup, S and O accumulators and P tile.
//   warp 0      TMA producer: the Q tiles once, then per step four 16-token pages of K and of V
//               (found through the block table) as 64-column panels with the 128-byte swizzle, two
//               stages each
//   warp 1      MMA issuer: per lane S = Q K^T (tcgen05.mma, M 128, N 64 keys, K = head_dim) into
//               one of the lane's two S accumulators in tensor memory, and O += P V (N = head_dim,
//               K = 64 keys, V read in place as an MN-major operand) into the lane's O accumulator.
//               S of step j+1 is issued before P V of step j, so the tensor cores work while step
//               j's softmax runs.
//   warps 2-5   softmax of lane 0 (warps 6-9: lane 1): thread i owns query row i. It reads its row
//               of S from tensor memory, applies the causal mask on the steps that touch the
//               diagonal, exponentiates against a running reference maximum, writes P (bf16) into
//               shared memory in the K-major
//               swizzled operand layout, and keeps the running sum. The reference maximum moves
//               only when a row's maximum has grown by more than 2^8 since it was set (then the O
//               row in tensor memory is rescaled in place), so most steps touch O not at all.
//               At the end the same threads normalise O and store it.
// Every wait is bounded; a wait that gives up sets the CTA's abort word, the roles leave their
// loops, tensor memory is freed and the status word is set.
//
// Replaces sdpa_prefill_mma_* / sdpa_prefill_nax_* (crates/rmlx-core/src/ops/sdpa.rs:1873-2855)
// with attention that reads the paged cache directly
// (crates/rmlx-nn/src/paged_kv_cache.rs:303-305 gathers on the CPU).
#include <cuda.h>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.cuh"

namespace rb {

constexpr int kTcRows = 128;                  // query rows per lane
constexpr int kTcKeys = 64;                   // keys per step
constexpr int kTcHd = 128;
constexpr int kTcPage = 16;
constexpr int kTcPages = kTcKeys / kTcPage;   // pages per step
constexpr int kTcQPanel = 128 * 128;          // 128 rows x 64 bf16 columns
constexpr int kTcQTile = 2 * kTcQPanel;       // 128 x 128 bf16
constexpr int kTcKvPanel = kTcKeys * 128;     // 64 rows x 64 bf16 columns
constexpr int kTcKvTile = 2 * kTcKvPanel;     // 64 x 128 bf16
constexpr int kTcPTile = kTcQPanel;           // 128 rows x 64 keys bf16
constexpr int kTcPageBytes = kTcPage * 128;   // one page inside a 64-column panel
constexpr float kTcRescaleStep = 8.f;         // log2 of the growth tolerated before O is rescaled

template <int LANES>
struct TcCfg {
  static constexpr int kThreads = 64 + 128 * LANES;
  // per lane: S0 [0,64) S1 [64,128); then per lane O (128 columns)
  static constexpr uint32_t kTmemCols = 256 * LANES;
  static constexpr int kBars = 9 + 6 * LANES;
  // Q per lane, K x2, V x2, P per lane, barriers. No slack for alignment: the kernel checks that
  // the dynamic shared-memory window starts on a 1024-byte boundary and refuses to run otherwise.
  static constexpr int kSmem = LANES * kTcQTile + 4 * kTcKvTile + LANES * kTcPTile + 256;
};

struct TcParams {
  const int* block_table;   // this sequence's pages
  __nv_bfloat16* out;       // [T, Hq, 128]
  int T, Hq, Hkv, pos0, n_qt;
  int window;               // > 0: a query sees only its last `window` keys
  float scale_log2;
  int* status;
};

__device__ __forceinline__ float tc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int LANES>
__global__ void __launch_bounds__(TcCfg<LANES>::kThreads, 1)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                        const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, TcParams p) {
  using C = TcCfg<LANES>;
  extern __shared__ __align__(1024) char smem[];
  if (smem_u32(smem) & 1023u) {       // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, kStatusBadArgument);
    return;
  }
  char* sQ = smem;                        // one tile per lane
  char* sK = sQ + LANES * kTcQTile;       // two stages
  char* sV = sK + 2 * kTcKvTile;          // two stages
  char* sP = sV + 2 * kTcKvTile;          // one tile per lane
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + LANES * kTcPTile);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;            // [2]
  uint64_t* k_free = bars + 3;            // [2]
  uint64_t* v_full = bars + 5;            // [2]
  uint64_t* v_free = bars + 7;            // [2]
  uint64_t* lane_bars = bars + 9;         // per lane: s_full[2], s_free[2], p_full, o_done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kBars);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // long rows of work first: the last query tile walks the most keys
  const int qt = p.n_qt - 1 - int(blockIdx.x) / p.Hq, h = int(blockIdx.x) % p.Hq;
  const int kvh = h / (p.Hq / p.Hkv);
  const int q0 = qt * (kTcRows * LANES);
  // steps of lane L: it sees keys [0, kv_end_L); a lane that starts past the last token is idle.
  // With a sliding window the block's steps start at j0, the step that holds the first key its
  // first row can see (later rows mask what lies before their own window).
  const int j0 = p.window > 0 ? max(0, p.pos0 + q0 - p.window + 1) / kTcKeys : 0;
  int n_steps[LANES];
  int n_max = 0, kv_end_max = 1;
#pragma unroll
  for (int L = 0; L < LANES; ++L) {
    const int first = q0 + L * kTcRows;
    const int kv_end = p.pos0 + min(first + kTcRows - 1, p.T - 1) + 1;
    n_steps[L] = first < p.T ? (kv_end + kTcKeys - 1) / kTcKeys - j0 : 0;
    if (n_steps[L] > 0) { n_max = max(n_max, n_steps[L]); kv_end_max = max(kv_end_max, kv_end); }
  }
  const int last_page = (kv_end_max - 1) / kTcPage;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + i, 1); mbar_init(k_free + i, 1);
      mbar_init(v_full + i, 1); mbar_init(v_free + i, 1);
    }
    for (int L = 0; L < LANES; ++L) {
      uint64_t* lb = lane_bars + 6 * L;
      mbar_init(lb + 0, 1); mbar_init(lb + 1, 1);     // s_full
      mbar_init(lb + 2, 4); mbar_init(lb + 3, 4);     // s_free: one arrival per softmax warp
      mbar_init(lb + 4, 4);                           // p_full
      mbar_init(lb + 5, 1);                           // o_done
    }
    // a wait that gave up earlier in this launch (or one the host has not cleared yet) ends the
    // remaining CTAs at their first wait instead of letting each run out its own polls
    *abort_flag = (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      pdl_wait();
      int last_k[2] = {-1, -1}, last_v[2] = {-1, -1};   // last step whose loads went to each stage
      const bool q_issued = *abort_flag == 0u;
      if (q_issued) {
        int active = 0;
#pragma unroll
        for (int L = 0; L < LANES; ++L) active += n_steps[L] > 0;
        mbar_arrive_expect_tx(q_full, active * kTcQTile);
#pragma unroll
        for (int L = 0; L < LANES; ++L) {
          if (n_steps[L] == 0) continue;
          tma_load_2d(sQ + L * kTcQTile, &tmap_q, q_full, h * kTcHd, q0 + L * kTcRows);
          tma_load_2d(sQ + L * kTcQTile + kTcQPanel, &tmap_q, q_full, h * kTcHd + 64, q0 + L * kTcRows);
        }
      }
      for (int j = 0; j < n_max; ++j) {
        if (*abort_flag) break;
        const int s = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        int y[kTcPages];
#pragma unroll
        for (int pg = 0; pg < kTcPages; ++pg) {
          // pages past the last one this CTA can see repeat it (their keys are masked)
          const int page = min((j + j0) * kTcPages + pg, last_page);
          y[pg] = (p.block_table[page] * p.Hkv + kvh) * kTcPage;
        }
        if (!mbar_wait(k_free + s, par, abort_flag)) break;
        mbar_arrive_expect_tx(k_full + s, kTcKvTile);
        last_k[s] = j;
        char* kd = sK + s * kTcKvTile;
#pragma unroll
        for (int pg = 0; pg < kTcPages; ++pg) {
          tma_load_2d(kd + pg * kTcPageBytes, &tmap_k, k_full + s, 0, y[pg]);
          tma_load_2d(kd + kTcKvPanel + pg * kTcPageBytes, &tmap_k, k_full + s, 64, y[pg]);
        }
        if (!mbar_wait(v_free + s, par, abort_flag)) break;
        mbar_arrive_expect_tx(v_full + s, kTcKvTile);
        last_v[s] = j;
        char* vd = sV + s * kTcKvTile;
#pragma unroll
        for (int pg = 0; pg < kTcPages; ++pg) {
          tma_load_2d(vd + pg * kTcPageBytes, &tmap_v, v_full + s, 0, y[pg]);
          tma_load_2d(vd + kTcKvPanel + pg * kTcPageBytes, &tmap_v, v_full + s, 64, y[pg]);
        }
      }
      if (*abort_flag) {
        // leaving early: let the copies already in flight land before the CTA gives up its
        // shared memory (they complete on their own; the polls are bounded all the same)
        auto drain = [](uint64_t* bar, uint32_t parity) {
          for (uint32_t i = 0; i < (1u << 16); ++i)
            if (mbar_try_wait(bar, parity)) return;
        };
        if (q_issued) drain(q_full, 0);
        for (int s = 0; s < 2; ++s) {
          if (last_k[s] >= 0) drain(k_full + s, (last_k[s] >> 1) & 1);
          if (last_v[s] >= 0) drain(v_full + s, (last_v[s] >> 1) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16_f32(128, kTcKeys);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(128, 128) | kUmmaBMajorMN;
      bool ok = mbar_wait(q_full, 0, abort_flag);
      // S of step j for every lane that still has work
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t u = (j >> 1) & 1;
        if (!mbar_wait(k_full + s, u, abort_flag)) return false;
        const uint32_t k_addr = smem_u32(sK + s * kTcKvTile);
#pragma unroll
        for (int L = 0; L < LANES; ++L) {
          if (j >= n_steps[L]) continue;
          uint64_t* lb = lane_bars + 6 * L;
          if (!mbar_wait(lb + 2 + s, u ^ 1u, abort_flag)) return false;   // s_free
          tc_fence_after_sync();
          const uint32_t q_addr = smem_u32(sQ + L * kTcQTile);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {       // 16 of the 128 head dimensions per product
            const uint32_t in_row = (ks & 3) * 32;
            tc_mma_f16(tmem_base + L * 128 + s * kTcKeys,
                       umma_desc_sw128_kmajor(q_addr + (ks >> 2) * kTcQPanel + in_row),
                       umma_desc_sw128_kmajor(k_addr + (ks >> 2) * kTcKvPanel + in_row), idesc_s,
                       ks != 0 ? 1u : 0u);
          }
          tc_commit(lb + s);                      // s_full
        }
        tc_commit(k_free + s);
        return true;
      };
      if (ok && n_max > 0) ok = issue_s(0);
      for (int j = 0; j < n_max && ok; ++j) {
        if (j + 1 < n_max && !issue_s(j + 1)) { ok = false; break; }
        const int s = j & 1;
        if (!mbar_wait(v_full + s, (j >> 1) & 1, abort_flag)) { ok = false; break; }
        const uint32_t v_addr = smem_u32(sV + s * kTcKvTile);
#pragma unroll
        for (int L = 0; L < LANES; ++L) {
          if (j >= n_steps[L]) continue;
          uint64_t* lb = lane_bars + 6 * L;
          if (!mbar_wait(lb + 4, j & 1, abort_flag)) { ok = false; break; }   // p_full
          tc_fence_after_sync();
          const uint32_t p_addr = smem_u32(sP + L * kTcPTile);
#pragma unroll
          for (int ks = 0; ks < kTcKeys / 16; ++ks) {       // 16 keys per product
            tc_mma_f16(tmem_base + LANES * 128 + L * 128, umma_desc_sw128_kmajor(p_addr + ks * 32),
                       umma_desc_sw128_mnmajor(v_addr + ks * 2048, kTcKvPanel), idesc_pv,
                       (j | ks) != 0 ? 1u : 0u);
          }
          tc_commit(lb + 5);                      // o_done
        }
        if (!ok) break;
        tc_commit(v_free + s);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups
    const int L = (warp - 2) >> 2;                     // lane served by this warpgroup
    const int quarter = warp & 3;                      // the 32 TMEM lanes this warp may touch
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = uint32_t(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + L * 128 + t_lane;
    const uint32_t tmem_o = tmem_base + LANES * 128 + L * 128 + t_lane;
    uint64_t* s_full = lane_bars + 6 * L;
    uint64_t* s_free = s_full + 2;
    uint64_t* p_full = s_full + 4;
    uint64_t* o_done = s_full + 5;
    const int lane_q0 = q0 + L * kTcRows;
    const int qrow = lane_q0 + row;
    const int pos = p.pos0 + qrow;
    const int my_steps = n_steps[LANES == 1 ? 0 : L];
    const float sc = p.scale_log2;
    char* prow = sP + L * kTcPTile + row * 128;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    pdl_wait();
#pragma unroll 1
    for (int j = 0; j < my_steps; ++j) {
      const int sb = j & 1;
      ok = mbar_wait(s_full + sb, (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      constexpr int NC = kTcKeys / 32;                 // 32-column chunks of this row of S
      uint32_t r[NC][32];
#pragma unroll
      for (int c = 0; c < NC; ++c) tmem_ld_32x32(tmem_s + sb * kTcKeys + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free + sb);         // the issuer may overwrite this S now

      const int k0 = (j + j0) * kTcKeys;
      if (k0 + kTcKeys - 1 > p.pos0 + lane_q0) {       // the step touches the diagonal
        const int vis = pos - k0;                      // keys k0 .. k0+vis are visible to this row
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > vis) r[c][i] = 0xff800000u;   // -inf
      }
      if (p.window > 0 && pos - p.window + 1 > k0) {   // keys before this row's window
        const int lo = pos - p.window + 1 - k0;        // keys k0 .. k0+lo-1 are out of the window
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < lo) r[c][i] = 0xff800000u;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[c][i]));
      const float m_new = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
      bool waited = false;
      if (__any_sync(0xffffffffu, m_new > m_used + kTcRescaleStep)) {
        const float m_next = fmaxf(m_used, m_new);
        const float alpha = (m_next == -INFINITY) ? 1.f : tc_ex2(m_used - m_next);
        l *= alpha;
        m_used = m_next;
        if (j > 0) {                                    // O holds steps 0..j-1: bring it to the new reference
          ok = mbar_wait(o_done, (j - 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          waited = true;
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + c * 32, o);
          }
          tmem_st_wait();
        }
      }
      const float sub = (m_used == -INFINITY) ? 0.f : m_used;
      uint32_t w[kTcKeys / 2];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = tc_ex2(fmaf(__uint_as_float(r[c][i]), sc, -sub));
          const float p1 = tc_ex2(fmaf(__uint_as_float(r[c][i + 1]), sc, -sub));
          sum4[(i >> 1) & 3] += p0 + p1;
          w[c * 16 + (i >> 1)] = pack_bf16(p0, p1);
        }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (j > 0 && !waited) {                           // P V of the previous step still reads sP
        ok = mbar_wait(o_done, (j - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < kTcKeys / 8; ++c)             // 16-byte chunks: 8 keys each
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) =
            make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && my_steps > 0) {
      ok = mbar_wait(o_done, (my_steps - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && my_steps > 0) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t(min(qrow, p.T - 1)) * p.Hq + h) * kTcHd;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_o + c * 32, o);
        tmem_ld_wait();
        if (qrow < p.T) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(o[v * 8]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = pk;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, kStatusMbarTimeout);
  pdl_launch_dependents();
}

template <int LANES>
static int launch_prefill_tc(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                             TcParams p, int pdl, cudaStream_t st) {
  auto kern = flash_prefill_tc_kernel<LANES>;
  constexpr size_t smem = TcCfg<LANES>::kSmem;
  RB_CHECK(set_max_smem(kern, smem));
  p.n_qt = (p.T + kTcRows * LANES - 1) / (kTcRows * LANES);
  return launch(kern, dim3(p.n_qt * p.Hq), dim3(TcCfg<LANES>::kThreads), smem, st, pdl != 0, tq, tk,
                tv, p);
}

}  // namespace rb

using namespace rb;

// 1 when the tensor-core kernel covers the shape (head_dim 128; any sliding window).
extern "C" int rmlx_flash_prefill_tc_supported(int HD, int window) {
  (void)window;
  return HD == kTcHd;
}

// q, out: [T, Hq, 128] bf16; caches [num_blocks, Hkv, 16, 128] bf16; block_table: the sequence's
// pages (int32, device); queries sit at positions pos0 .. pos0+T-1 and the cache already holds keys
// 0 .. pos0+T-1. window > 0: sliding-window attention over the last `window` keys. lanes: query tiles per CTA, 1 or 2 (0 = choose; one tile measured at least as
// fast as two at every length tried, so that is the choice). status: optional device int set
// non-zero if a pipeline wait gave up.
extern "C" int rmlx_flash_prefill_tc(const void* q, const void* k_cache, const void* v_cache,
                                     const int* block_table, void* out, int T, int Hq, int Hkv,
                                     int HD, int num_blocks, int pos0, int window, float scale,
                                     int lanes, int* status, int pdl, cudaStream_t st) {
  if (T < 1 || HD != kTcHd || Hkv < 1 || Hq % Hkv || pos0 < 0 || num_blocks < 1) return -2;
  if (lanes == 0) lanes = 1;
  if (lanes != 1 && lanes != 2) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out)) & 15)
    return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d_bf16(&tq, q, uint64_t(Hq) * kTcHd, uint64_t(T), uint64_t(Hq) * kTcHd * 2, 64,
                             kTcRows);
  if (rc) return rc;
  const uint64_t rows = uint64_t(num_blocks) * Hkv * kTcPage;
  rc = make_tmap_2d_bf16(&tk, k_cache, kTcHd, rows, kTcHd * 2, 64, kTcPage);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v_cache, kTcHd, rows, kTcHd * 2, 64, kTcPage);
  if (rc) return rc;
  TcParams p;
  p.block_table = block_table;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.pos0 = pos0;
  p.n_qt = 0;
  p.window = window > 0 ? window : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  return lanes == 2 ? launch_prefill_tc<2>(tq, tk, tv, p, pdl, st)
                    : launch_prefill_tc<1>(tq, tk, tv, p, pdl, st);
}
