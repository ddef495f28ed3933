// Decode attention for multi-head latent attention over a PAGED LATENT cache.
//
// The cache holds, per token, the compressed latent c_kv (LAT values) followed by the decoupled
// RoPE key (ROPE values): one row of LAT + ROPE bf16 shared by all heads
// (crates/rmlx-nn/src/mla.rs:111-250, MlaKvCache). With the key up-projection absorbed into the
// query (q_lat = q_nope W_uk per head) the attention of one new token is
//     score[h, t] = scale * (q_lat[h] . c_kv[t] + q_rope[h] . k_rope[t])
//     o_lat[h]    = sum_t softmax(score)[h, t] * c_kv[t]
// i.e. flash decode with one KV "head" of width LAT + ROPE for the keys and LAT for the values,
// shared by every query head; the value up-projection follows outside. Nothing is expanded per
// head in memory: a cached token costs (LAT + ROPE) * 2 bytes whatever the number of heads.
//
// One block = (KV split, tile of 16 query heads, sequence). The block's four warps all walk the
// same pages (a block-wide ring of cp.async stages); each computes the 16 x 16 score tile with
// mma.sync (queries from shared memory, keys straight from the staged page) and owns a quarter of
// the LAT output columns for the P V product. Splits are merged by a second small kernel.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kMlaPage = 16;
constexpr int kMlaWarps = 4;
constexpr int kMlaThreads = kMlaWarps * 32;
constexpr int kMlaStages = 3;

__device__ __forceinline__ void mla_cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void mla_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void mla_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
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
  const __nv_bfloat16* cache;    // [blocks, 16, LAT + ROPE]
  const int* block_table;        // [B, max_blocks]
  const int* seq_lens;           // [B] tokens in the cache including the current one
  __nv_bfloat16* out;            // [B, H, LAT]
  float* part_o;                 // [B, HT, S, 16, LAT]
  float* part_ml;                // [B, HT, S, 16, 2]
  int max_blocks, H, HT, S;
  float scale_log2;
};

// Row layout in shared memory (queries and pages alike): row r is (LAT + ROPE) * 2 bytes, its
// 16-byte chunk c sits at chunk position c ^ (r & 7), which keeps ldmatrix conflict-free.
template <int LAT, int ROPE>
__global__ void __launch_bounds__(kMlaThreads) mla_decode_kernel(MlaParams p) {
  constexpr int W = LAT + ROPE;            // values per row
  constexpr int CH = W / 8;                // 16-byte chunks per row
  constexpr int KS = W / 16;               // k-steps of the score product
  constexpr int NTW = LAT / kMlaWarps / 8; // output n-tiles per warp
  constexpr int ROW_BYTES = W * 2;
  constexpr int PAGE_BYTES = kMlaPage * ROW_BYTES;
  static_assert(CH % 8 == 0 && LAT % (kMlaWarps * 16) == 0, "widths: multiples of 64 / 64");
  extern __shared__ __align__(128) char smem[];
  char* qs = smem;                              // 16 query rows
  char* ring = smem + PAGE_BYTES;               // kMlaStages pages

  const int split = blockIdx.x, ht = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();
  pdl_wait();
  const int len = p.seq_lens[b];
  const int pg_total = (len + kMlaPage - 1) / kMlaPage;
  const int per = (pg_total + p.S - 1) / p.S;
  const int pg0 = split * per, pg1 = min(pg0 + per, pg_total);
  const int* bt = p.block_table + size_t(b) * p.max_blocks;

  auto issue = [&](int pg, int stage) {
    const int blk = RB_BOUNDS(pg, p.max_blocks) ? bt[pg] : 0;
    const char* src = reinterpret_cast<const char*>(p.cache) + size_t(blk) * PAGE_BYTES;
    char* dst = ring + stage * PAGE_BYTES;
    for (int idx = threadIdx.x; idx < kMlaPage * CH; idx += kMlaThreads) {
      const int r = idx / CH, c = idx - r * CH;
      mla_cp_async16(dst + r * ROW_BYTES + (((c & ~7) | ((c ^ r) & 7)) << 4), src + idx * 16);
    }
  };
  // queries of this head tile (rows beyond H are zero)
  for (int idx = threadIdx.x; idx < 16 * CH; idx += kMlaThreads) {
    const int r = idx / CH, c = idx - r * CH;
    const int h = ht * 16 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (h < p.H) v = *reinterpret_cast<const uint4*>(p.q + (size_t(b) * p.H + h) * W + c * 8);
    *reinterpret_cast<uint4*>(qs + r * ROW_BYTES + (((c & ~7) | ((c ^ r) & 7)) << 4)) = v;
  }
#pragma unroll
  for (int s = 0; s < kMlaStages; ++s) {
    if (pg0 + s < pg1) issue(pg0 + s, s);
    mla_cp_commit();
  }

  float o[NTW][4];
#pragma unroll
  for (int j = 0; j < NTW; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const uint32_t qbase = smem_u32(qs);
  int stage = 0;
  for (int pg = pg0; pg < pg1; ++pg) {
    mla_cp_wait<kMlaStages - 1>();
    __syncthreads();                         // the page (and, first time, the queries) are visible
    const uint32_t kbase = smem_u32(ring + stage * PAGE_BYTES);
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int ks = 0; ks < KS; ++ks) {
      const int mi = lane >> 3, r = lane & 7;
      uint32_t qa[4], kb[4];
      {   // A: rows = heads; matrices (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        const int row = (mi & 1) * 8 + r, c = 2 * ks + (mi >> 1);
        mla_ldm_x4(qa, qbase + row * ROW_BYTES + (((c & ~7) | ((c ^ row) & 7)) << 4));
      }
      {   // B: rows = tokens; matrices (tok 0-7, k lo), (tok 0-7, k hi), (tok 8-15, k lo), (tok 8-15, k hi)
        const int tok = (mi >> 1) * 8 + r, c = 2 * ks + (mi & 1);
        mla_ldm_x4(kb, kbase + tok * ROW_BYTES + (((c & ~7) | ((c ^ tok) & 7)) << 4));
      }
      mla_mma(s0, qa, kb[0], kb[1]);
      mla_mma(s1, qa, kb[2], kb[3]);
    }
    const int tok0 = pg * kMlaPage + t * 2;
    float sv[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};
    const int tk[4] = {tok0, tok0 + 1, tok0 + 8, tok0 + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = tk[i] < len;
      sv[i] = ok ? sv[i] * p.scale_log2 : -INFINITY;
      sv[4 + i] = ok ? sv[4 + i] * p.scale_log2 : -INFINITY;
    }
    float mx0 = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    float mx1 = fmaxf(fmaxf(sv[4], sv[5]), fmaxf(sv[6], sv[7]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);   // finite: a page holds a visible token
    const float c0 = exp2f(m0 - nm0), c1 = exp2f(m1 - nm1);
    m0 = nm0; m1 = nm1;
    float pr[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) { pr[i] = exp2f(sv[i] - m0); pr[4 + i] = exp2f(sv[4 + i] - m1); }
    l0 = l0 * c0 + (pr[0] + pr[1] + pr[2] + pr[3]);
    l1 = l1 * c1 + (pr[4] + pr[5] + pr[6] + pr[7]);
    const uint32_t pa[4] = {pack_bf16(pr[0], pr[1]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[2], pr[3]),
                            pack_bf16(pr[6], pr[7])};
#pragma unroll
    for (int j = 0; j < NTW; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V over this warp's quarter of the latent columns
#pragma unroll
    for (int j = 0; j < NTW; j += 2) {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = (mi & 1) * 8 + r, c = warp * NTW + j + (mi >> 1);
      uint32_t vb[4];
      mla_ldm_x4_trans(vb, kbase + tok * ROW_BYTES + (((c & ~7) | ((c ^ tok) & 7)) << 4));
      mla_mma(o[j], pa, vb[0], vb[1]);
      mla_mma(o[j + 1], pa, vb[2], vb[3]);
    }
    __syncthreads();                         // every warp is done with this stage
    if (pg + kMlaStages < pg1) issue(pg + kMlaStages, stage);
    mla_cp_commit();
    stage = (stage + 1 == kMlaStages) ? 0 : stage + 1;
  }
  mla_cp_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

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

// One block per (sequence, head tile): weights exp2(m_s - M) / L per split and row, then the sum.
template <int LAT>
__global__ void __launch_bounds__(256) mla_merge_kernel(MlaParams p) {
  __shared__ float wgt[64 * 16];
  const int ht = blockIdx.x, b = blockIdx.y;
  pdl_launch_dependents();
  pdl_wait();
  const size_t tile0 = (size_t(b) * p.HT + ht) * p.S;
  if (threadIdx.x < 16) {
    const int row = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < p.S; ++s) M = fmaxf(M, p.part_ml[((tile0 + s) * 16 + row) * 2]);
    float L = 0.f;
    for (int s = 0; s < p.S; ++s) {
      const float ms = p.part_ml[((tile0 + s) * 16 + row) * 2];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      wgt[s * 16 + row] = f;
      L += p.part_ml[((tile0 + s) * 16 + row) * 2 + 1] * f;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int s = 0; s < p.S; ++s) wgt[s * 16 + row] *= inv;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * (LAT / 2); idx += 256) {
    const int row = idx / (LAT / 2), d = (idx - row * (LAT / 2)) * 2;
    const int h = ht * 16 + row;
    if (h >= p.H) continue;
    float a0 = 0.f, a1 = 0.f;
    for (int s = 0; s < p.S; ++s) {
      const float2 v = *reinterpret_cast<const float2*>(p.part_o + ((tile0 + s) * 16 + row) * LAT + d);
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

// q [B, H, LAT + ROPE] bf16 (absorbed), cache [blocks, 16, LAT + ROPE] bf16, out [B, H, LAT] bf16.
// (LAT, ROPE) in {(512, 64), (128, 64)}; splits in [1, 64]; part_* needed when splits > 1.
extern "C" int rmlx_mla_decode_paged(const void* q, const void* cache, const int* block_table,
                                     const int* seq_lens, void* out, float* part_o, float* part_ml,
                                     int B, int H, int LAT, int ROPE, int max_blocks, int splits,
                                     float scale, int pdl, cudaStream_t st) {
  if (B < 1 || H < 1 || splits < 1 || splits > 64) return -2;
  if (splits > 1 && (!part_o || !part_ml)) return -2;
  MlaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.cache = static_cast<const __nv_bfloat16*>(cache);
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml;
  p.max_blocks = max_blocks; p.H = H; p.HT = (H + 15) / 16; p.S = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(splits, p.HT, B);
#define RB_MLA(LAT_, ROPE_)                                                                   \
  {                                                                                           \
    const size_t smem = size_t(1 + kMlaStages) * kMlaPage * (LAT_ + ROPE_) * 2;               \
    auto kern = mla_decode_kernel<LAT_, ROPE_>;                                               \
    RB_CHECK(set_max_smem(kern, smem));                                                       \
    int rc = launch(kern, grid, dim3(kMlaThreads), smem, st, pdl != 0, p);                    \
    if (rc || splits == 1) return rc;                                                         \
    return launch(mla_merge_kernel<LAT_>, dim3(p.HT, B), dim3(256), 0, st, pdl != 0, p);      \
  }
  if (LAT == 512 && ROPE == 64) RB_MLA(512, 64)
  if (LAT == 128 && ROPE == 64) RB_MLA(128, 64)
#undef RB_MLA
  return -2;
}
