// Decode attention for multi-head latent attention over a PAGED LATENT cache.
//
// The cache holds, per token, the compressed latent c_kv (LAT values) followed by the decoupled
// RoPE key (ROPE values) and 8 values of padding: one row of LAT + ROPE + 8 bf16 shared by all heads
// (crates/rmlx-nn/src/mla.rs:111-250, MlaKvCache). With the key up-projection absorbed into the
// query (q_lat = q_nope W_uk per head) the attention of one new token is
//     score[h, t] = scale * (q_lat[h] . c_kv[t] + q_rope[h] . k_rope[t])
//     o_lat[h]    = sum_t softmax(score)[h, t] * c_kv[t]
// i.e. flash decode with one KV "head" of width LAT + ROPE for the keys and LAT for the values,
// shared by every query head; the value up-projection follows outside. Nothing is expanded per
// head in memory: a cached token costs (LAT + ROPE) * 2 bytes whatever the number of heads.
//
// One block = (KV split, tile of 16 query heads, sequence); eight warps. The block walks its share
// of the sequence in steps of four pages (64 tokens), double-buffered: one warp issues ONE bulk copy
// (cp.async.bulk, completing on an mbarrier) per page. A bulk copy occupies the copy engine for
// about as long whatever its size, so a page of 18 KB must not be fetched row by row; the 16 bytes
// of padding that keep ldmatrix conflict-free without a swizzle are therefore part of the cache's
// row in global memory, and a page lands in shared memory as it is. Within a step warp w computes the
// 16 heads x 8 tokens score tile of tokens 8w .. 8w+7 with mma.sync (queries from shared memory,
// keys straight from the staged page), the warps agree on the step's row maxima through shared
// memory, every warp writes its probabilities (bf16) into a shared 16 x 64 tile, and then each
// warp runs the P V product over all 64 tokens for its eighth of the LAT output columns. No score
// is computed twice. Splits are merged by a second kernel.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kMlaPage = 16;
constexpr int kMlaStages = 2;

__device__ int g_mla_status = 0;          // kStatusMbarTimeout once a wait for staged pages gave up

__device__ __forceinline__ void mla_bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void mla_ldm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mla_ldm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mla_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct MlaParams {
  const __nv_bfloat16* q;        // [B, H, LAT + ROPE]  absorbed query: q_lat then q_rope
  const __nv_bfloat16* cache;    // [blocks, 16, LAT + ROPE + 8]
  const int* block_table;        // [slots, max_blocks]
  const int* seq_lens;           // [slots] tokens in the cache including the current one
  const int* slots;              // [B] cache slot of each query row (null: row b uses slot b)
  __nv_bfloat16* out;            // [B, H, LAT]
  float* part_o;                 // [B, HT, S, 16, LAT]
  float* part_ml;                // [B, HT, S, 16, 2]
  int max_blocks, H, HT, S;
  float scale_log2;
};

// Shared memory: rows of queries and staged pages are (LAT + ROPE) * 2 + 16 bytes apart (eight
// consecutive rows start in eight different 16-byte bank groups). The probability tile is 16 rows
// of 64 bf16 whose 16-byte chunk c sits at position c ^ (row & 7).
// WARPS = 8: steps of 64 tokens, one block per SM (the choice while the grid fits the SMs once).
// WARPS = 4: steps of 32 tokens at half the shared memory, so two blocks share an SM and one
// block's exchange / softmax phases overlap the other's tensor-core phases.
template <int LAT, int ROPE, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 4 ? 2 : 1) mla_decode_kernel(MlaParams p) {
  constexpr int kMlaWarps = WARPS, kMlaThreads = WARPS * 32;
  constexpr int kMlaStepPages = WARPS / 2;   // eight tokens per warp in the score product
  constexpr int W = LAT + ROPE;            // values per row
  constexpr int CH = W / 8;                // 16-byte chunks per row
  constexpr int KS = W / 16;               // k-steps of the score product
  constexpr int NTW = LAT / kMlaWarps / 8; // output n-tiles per warp
  constexpr int ROW_BYTES = W * 2;
  constexpr int ROW_PAD = ROW_BYTES + 16;
  constexpr int PAGE_SM = kMlaPage * ROW_PAD;
  constexpr int STEP_SM = kMlaStepPages * PAGE_SM;
  constexpr int STEP_ROWS = kMlaStepPages * kMlaPage;
  static_assert(KS % 4 == 0 && NTW % 2 == 0 && NTW >= 2, "widths: LAT a multiple of 128, LAT + ROPE of 64");
  static_assert(STEP_ROWS == 8 * kMlaWarps, "eight tokens per warp");
  static_assert(PAGE_SM % 128 == 0, "tiles stay 128-byte aligned");
  extern __shared__ __align__(128) char smem[];
  char* qs = smem;                                        // 16 query rows
  char* ring = smem + PAGE_SM;                            // kMlaStages steps of four pages
  char* ps = ring + kMlaStages * STEP_SM;                 // probabilities [16][<= 64] bf16, 128-byte rows
  float* red = reinterpret_cast<float*>(ps + 16 * 128);   // [warps][16] row maxima / row sums
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + kMlaWarps * 16);   // one per stage

  const int split = blockIdx.x, ht = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  if (threadIdx.x == 0) {
    mbar_init(bars, 1);
    mbar_init(bars + 1, 1);
    fence_mbar_init();
  }
  pdl_launch_dependents();
  pdl_wait();
  const int slot = p.slots ? p.slots[b] : b;
  const int len = p.seq_lens[slot];
  const int pg_total = (len + kMlaPage - 1) / kMlaPage;
  const int per = ((pg_total + p.S - 1) / p.S + kMlaStepPages - 1) / kMlaStepPages * kMlaStepPages;
  const int pg0 = split * per, pg1 = min(pg0 + per, pg_total);
  const int steps = pg1 > pg0 ? (pg1 - pg0 + kMlaStepPages - 1) / kMlaStepPages : 0;
  const int* bt = p.block_table + size_t(slot) * p.max_blocks;

  // Warp 0 stages the pages of step `st`: lane i copies page i whole. A page past the split's end
  // is filled with zeros so that its (zero-probability) rows cannot bring a NaN into the P V
  // product. The block ids of a step are read from the block table one step before they are
  // needed (`load_id`), which keeps that read off the copy's critical path.
  auto load_id = [&](int st) -> int {
    const int pg = pg0 + st * kMlaStepPages + lane;
    return (lane < kMlaStepPages && pg < pg1 && RB_BOUNDS(pg, p.max_blocks)) ? bt[pg] : 0;
  };
  auto issue = [&](int st, int stage, int id) {
    const int first = pg0 + st * kMlaStepPages;
    const int valid = min(kMlaStepPages, pg1 - first);
    if (lane == 0) mbar_arrive_expect_tx(bars + stage, uint32_t(valid) * PAGE_SM);
    __syncwarp();
    char* dst = ring + stage * STEP_SM;
    if (lane < valid)
      mla_bulk_g2s(smem_u32(dst + lane * PAGE_SM), reinterpret_cast<const char*>(p.cache) + size_t(id) * PAGE_SM,
                   PAGE_SM, bars + stage);
    for (int idx = valid * (PAGE_SM / 16) + lane; idx < kMlaStepPages * (PAGE_SM / 16); idx += 32)
      *reinterpret_cast<uint4*>(dst + idx * 16) = make_uint4(0u, 0u, 0u, 0u);
  };
  // queries of this head tile (rows beyond H are zero)
  for (int idx = threadIdx.x; idx < 16 * CH; idx += kMlaThreads) {
    const int r = idx / CH, c = idx - r * CH;
    const int h = ht * 16 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (h < p.H) v = *reinterpret_cast<const uint4*>(p.q + (size_t(b) * p.H + h) * W + c * 8);
    *reinterpret_cast<uint4*>(qs + r * ROW_PAD + c * 16) = v;
  }
  __syncthreads();              // the barriers are initialised, the queries staged
  int id_next = 0;                        // warp 0, lane i: block id of page i of the step issued next
  if (warp == 0 && steps > 0) {
    const int id0 = load_id(0);
    id_next = load_id(1);
    issue(0, 0, id0);
  }

  float o[NTW][4];
#pragma unroll
  for (int j = 0; j < NTW; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // l: this warp's tokens only
  const int mi = lane >> 3, r8 = lane & 7;
  // per-lane ldmatrix bases; everything added to them below is a compile-time constant
  const uint32_t q_lane = smem_u32(qs) + ((mi & 1) * 8 + r8) * ROW_PAD + (mi >> 1) * 16;
  const uint32_t k_lane = ((warp & 1) * 8 + r8) * ROW_PAD + mi * 16 + (warp >> 1) * PAGE_SM;
  const uint32_t v_lane = ((mi & 1) * 8 + r8) * ROW_PAD + (warp * NTW + (mi >> 1)) * 16;
  const uint32_t p_lane = smem_u32(ps) + ((mi & 1) * 8 + r8) * 128;
  const uint32_t p_x = uint32_t((mi >> 1) ^ r8);          // chunk (2 kk + mi>>1) ^ r8 = (2 kk) ^ p_x
  bool timed_out = false;
  for (int st = 0; st < steps; ++st) {
    const int stage = st & 1;
    {   // bounded wait for the staged step; each thread observes the completed phase itself
      bool ok = false;
      for (uint32_t i = 0; i < kMbarPollLimit; ++i) {
        if (mbar_try_wait(bars + stage, uint32_t(st >> 1) & 1u)) { ok = true; break; }
      }
      timed_out |= !ok;
    }
    __syncthreads();            // every warp has left step st - 1: its stage may be refilled
    if (warp == 0 && st + 1 < steps) {
      issue(st + 1, stage ^ 1, id_next);
      id_next = load_id(st + 2);
    }
    const uint32_t sbase = smem_u32(ring + stage * STEP_SM);
    // scores of this warp's eight tokens: four independent accumulator chains
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ks += 4) {
      uint32_t kb[2][4], qa[4];
      mla_ldm_x4(kb[0], sbase + k_lane + ks * 32);          // (k lo, k hi) of ks, then of ks + 1
      mla_ldm_x4(kb[1], sbase + k_lane + (ks + 2) * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // A: rows = heads; matrices (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        mla_ldm_x4(qa, q_lane + (ks + i) * 32);
        mla_mma(s[i], qa, kb[i >> 1][(i & 1) * 2], kb[i >> 1][(i & 1) * 2 + 1]);
      }
    }
    const int pg = pg0 + st * kMlaStepPages + (warp >> 1);
    const int tok0 = pg * kMlaPage + (warp & 1) * 8 + t * 2;
    float sv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = pg < pg1 && tok0 + (i & 1) < len;
      sv[i] = ok ? (s[0][i] + s[1][i] + s[2][i] + s[3][i]) * p.scale_log2 : -INFINITY;
    }
    float mx0 = fmaxf(sv[0], sv[1]), mx1 = fmaxf(sv[2], sv[3]);   // rows g and g + 8
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (t == 0) { red[warp * 16 + g] = mx0; red[warp * 16 + g + 8] = mx1; }
    __syncthreads();            // the eight warps' row maxima
#pragma unroll
    for (int w = 0; w < kMlaWarps; ++w) {
      mx0 = fmaxf(mx0, red[w * 16 + g]);
      mx1 = fmaxf(mx1, red[w * 16 + g + 8]);
    }
    // finite: the step's first page holds a visible token
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    const float c0 = exp2f(m0 - nm0), c1 = exp2f(m1 - nm1);
    m0 = nm0; m1 = nm1;
    const float p0 = exp2f(sv[0] - m0), p1 = exp2f(sv[1] - m0), p2 = exp2f(sv[2] - m1), p3 = exp2f(sv[3] - m1);
    l0 = l0 * c0 + (p0 + p1);
    l1 = l1 * c1 + (p2 + p3);
    // this warp's eight columns of the probability tile are chunk `warp` of each row
    *reinterpret_cast<uint32_t*>(ps + g * 128 + ((warp ^ g) << 4) + 4 * t) = pack_bf16(p0, p1);
    *reinterpret_cast<uint32_t*>(ps + (g + 8) * 128 + ((warp ^ g) << 4) + 4 * t) = pack_bf16(p2, p3);
#pragma unroll
    for (int j = 0; j < NTW; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    __syncthreads();            // the probability tile is complete
    // O += P V over the step's 64 tokens and this warp's share of the latent columns
#pragma unroll
    for (int kk = 0; kk < kMlaStepPages; ++kk) {
      uint32_t pa[4];
      mla_ldm_x4(pa, p_lane + ((uint32_t(2 * kk) ^ p_x) << 4));
#pragma unroll
      for (int j = 0; j < NTW; j += 2) {
        uint32_t vb[4];
        mla_ldm_x4_trans(vb, sbase + v_lane + kk * PAGE_SM + j * 16);
        mla_mma(o[j], pa, vb[0], vb[1]);
        mla_mma(o[j + 1], pa, vb[2], vb[3]);
      }
    }
  }
  if (timed_out) atomicExch(&g_mla_status, int(kStatusMbarTimeout));
  // row sums: over the quad, then over the warps (all share the same running maximum)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();              // the last step's reads of `red` are over
  if (t == 0) { red[warp * 16 + g] = l0; red[warp * 16 + g + 8] = l1; }
  __syncthreads();
  l0 = l1 = 0.f;
#pragma unroll
  for (int w = 0; w < kMlaWarps; ++w) { l0 += red[w * 16 + g]; l1 += red[w * 16 + g + 8]; }

  const size_t tile = (size_t(b) * p.HT + ht) * p.S + split;
#pragma unroll
  for (int j = 0; j < NTW; ++j) {
    const int d = (warp * NTW + j) * 8 + t * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = g + half * 8, h = ht * 16 + row;
      const float v0 = o[j][half * 2], v1 = o[j][half * 2 + 1], L = half ? l1 : l0;
      if (p.S == 1) {
        if (h < p.H) {
          const float inv = L > 0.f ? 1.f / L : 0.f;
          *reinterpret_cast<uint32_t*>(p.out + (size_t(b) * p.H + h) * LAT + d) = pack_bf16(v0 * inv, v1 * inv);
        }
      } else {
        *reinterpret_cast<float2*>(p.part_o + (tile * 16 + row) * LAT + d) = make_float2(v0, v1);
      }
    }
  }
  if (p.S > 1 && warp == 0 && t == 0) {
    p.part_ml[(tile * 16 + g) * 2] = m0;     p.part_ml[(tile * 16 + g) * 2 + 1] = l0;
    p.part_ml[(tile * 16 + g + 8) * 2] = m1; p.part_ml[(tile * 16 + g + 8) * 2 + 1] = l1;
  }
  pdl_launch_dependents();
}

// One block per (sequence, head tile, 64 output columns). Weights exp2(m_s - M) / L per split and
// row first (16 lanes per row, up to four splits per lane), then the weighted sum of the partials.
template <int LAT>
__global__ void __launch_bounds__(256) mla_merge_kernel(MlaParams p) {
  __shared__ float wgt[64 * 16];
  const int ht = blockIdx.x, b = blockIdx.y, cz = blockIdx.z;
  pdl_launch_dependents();
  pdl_wait();
  const size_t tile0 = (size_t(b) * p.HT + ht) * p.S;
  {
    const int row = threadIdx.x >> 4, ls = threadIdx.x & 15;
    float ms[4], lsum[4], M = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int s = ls + 16 * k;
      ms[k] = -INFINITY; lsum[k] = 0.f;
      if (s < p.S) {
        const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + ((tile0 + s) * 16 + row) * 2);
        ms[k] = ml.x; lsum[k] = ml.y;
      }
      M = fmaxf(M, ms[k]);
    }
#pragma unroll
    for (int off = 8; off; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float f[4], L = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[k] = (ms[k] == -INFINITY) ? 0.f : exp2f(ms[k] - M);
      L += lsum[k] * f[k];
    }
#pragma unroll
    for (int off = 8; off; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int s = ls + 16 * k;
      if (s < p.S) wgt[s * 16 + row] = f[k] * inv;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int idx = threadIdx.x + 256 * i;              // 16 rows x 32 column pairs
    const int row = idx >> 5, d = cz * 64 + (idx & 31) * 2;
    const int h = ht * 16 + row;
    if (h >= p.H) continue;
    const float* src = p.part_o + (tile0 * 16 + row) * LAT + d;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
    for (int s = 0; s < p.S; ++s) {
      const float2 v = *reinterpret_cast<const float2*>(src + size_t(s) * 16 * LAT);
      const float w = wgt[s * 16 + row];
      a0 = fmaf(v.x, w, a0); a1 = fmaf(v.y, w, a1);
    }
    *reinterpret_cast<uint32_t*>(p.out + (size_t(b) * p.H + h) * LAT + d) = pack_bf16(a0, a1);
  }
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("mla_decode.cu")

extern "C" long long rmlx_mla_decode_part_o_elems(int B, int H, int S, int LAT) {
  return 1LL * B * ((H + 15) / 16) * S * 16 * LAT;
}
extern "C" long long rmlx_mla_decode_part_ml_elems(int B, int H, int S) {
  return 1LL * B * ((H + 15) / 16) * S * 16 * 2;
}

// 0 while every wait for staged pages completed; kStatusMbarTimeout otherwise. Reading resets it.
extern "C" int rmlx_mla_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_mla_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_mla_status, &zero, sizeof(int));
  return v;
}

// q [B, H, LAT + ROPE] bf16 (absorbed), cache [blocks, 16, row_elems = LAT + ROPE + 8] bf16 (the
// last 8 values of a row are padding), out [B, H, LAT] bf16.
// block_table / seq_lens are the cache's own tables, indexed by slots[b] (by b when slots is null).
// (LAT, ROPE) in {(512, 64), (128, 64)}; splits in [1, 64]; part_* needed when splits > 1.
extern "C" int rmlx_mla_decode_paged(const void* q, const void* cache, const int* block_table,
                                     const int* seq_lens, const int* slots, void* out, float* part_o, float* part_ml,
                                     int B, int H, int LAT, int ROPE, int row_elems, int max_blocks,
                                     int splits, float scale, int pdl, cudaStream_t st) {
  if (B < 1 || H < 1 || splits < 1 || splits > 64) return -2;
  if (row_elems != LAT + ROPE + 8) return -2;     // the padded row layout is part of the contract
  if (splits > 1 && (!part_o || !part_ml)) return -2;
  MlaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.block_table = block_table; p.seq_lens = seq_lens; p.slots = slots;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml;
  p.max_blocks = max_blocks; p.H = H; p.HT = (H + 15) / 16; p.S = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(splits, p.HT, B);
  const bool narrow = 1LL * splits * p.HT * B > 148;   // more blocks than SMs: two narrow blocks per SM
#define RB_MLA(LAT_, ROPE_)                                                                   \
  {                                                                                           \
    const int warps = narrow ? 4 : 8;                                                         \
    const size_t smem = size_t(1 + kMlaStages * (warps / 2)) * kMlaPage * ((LAT_ + ROPE_) * 2 + 16) \
                        + 16 * 128 + warps * 16 * sizeof(float) + kMlaStages * 8;             \
    auto kern = narrow ? mla_decode_kernel<LAT_, ROPE_, 4> : mla_decode_kernel<LAT_, ROPE_, 8>; \
    RB_CHECK(set_max_smem(kern, smem));                                                       \
    int rc = launch(kern, grid, dim3(warps * 32), smem, st, pdl != 0, p);                     \
    if (rc || splits == 1) return rc;                                                         \
    return launch(mla_merge_kernel<LAT_>, dim3(p.HT, B, LAT_ / 64), dim3(256), 0, st, pdl != 0, p); \
  }
  if (LAT == 512 && ROPE == 64) RB_MLA(512, 64)
  if (LAT == 128 && ROPE == 64) RB_MLA(128, 64)
#undef RB_MLA
  return -2;
}
