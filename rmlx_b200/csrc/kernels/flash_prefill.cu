// Paged causal flash attention for prompt processing (many query tokens of one sequence).
//
// A block owns 64 query tokens of one query head (four warps x 16 rows); K and V come from the
// paged cache through the block table, 64 keys (four pages) at a time, staged once per block with
// a two-stage cp.async pipeline into swizzled shared memory and shared by the four warps. Each warp
// runs the online-softmax recurrence on m16n8k16 tensor-core tiles (QK^T, then PV with P re-used
// from the accumulator registers). Tiles entirely above the diagonal are skipped; the diagonal
// tile is masked per element; a sliding window adds a lower bound. Works for chunked prefill and
// prefix reuse: queries sit at positions pos0 .. pos0+T-1 and see every cached key at or before
// their own position.
//
// This is the mma.sync form; the query/key products of a 64-row block do not fill a tcgen05 tile
// pair without restructuring the softmax around tensor memory, which is left as the next step.
//
// Replaces sdpa_prefill_mma_* / sdpa_prefill_nax_* over contiguous slabs
// (crates/rmlx-core/src/ops/sdpa.rs:1873-2855) and adds what the reference lacks: attention that
// reads the paged cache directly (crates/rmlx-nn/src/paged_kv_cache.rs:303-305 gathers on the CPU).
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kFpPage = 16;
constexpr int kFpWarps = 4;
constexpr int kFpThreads = 128;
constexpr int kFpKvTile = 64;   // keys per staged tile = 4 pages

__device__ __forceinline__ void fp_cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void fp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fp_ldm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fp_ldm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fp_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct FpParams {
  const __nv_bfloat16* q;        // [T, Hq, HD]
  const __nv_bfloat16* k_cache;  // [blocks, Hkv, 16, HD]
  const __nv_bfloat16* v_cache;
  const int* block_table;        // this sequence's row
  __nv_bfloat16* out;            // [T, Hq, HD]
  int T, Hq, Hkv, pos0, window;
  float scale_log2;
};

template <int HD>
__global__ void __launch_bounds__(kFpThreads) flash_prefill_kernel(FpParams p) {
  constexpr int CH = HD / 8, KS = HD / 16, NT = HD / 8;
  constexpr int PAGE_BYTES = kFpPage * HD * 2;
  constexpr int TILE_BYTES = 4 * PAGE_BYTES;           // 64 keys
  extern __shared__ __align__(128) char smem[];        // 2 stages x (K tile, V tile)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int qt = blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.Hq / p.Hkv);
  pdl_wait();
  const int q0 = qt * 64;                               // first query token of the block
  const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;   // this lane's two query tokens
  const int pos_a = p.pos0 + row_a, pos_b = p.pos0 + row_b;
  const int last_q = min(q0 + 63, p.T - 1);
  const int kv_end = p.pos0 + last_q + 1;               // keys needed by this block: [kv_begin, kv_end)
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, p.pos0 + q0 - p.window + 1);
  const int tile_begin = kv_begin / kFpKvTile, tile_end = (kv_end + kFpKvTile - 1) / kFpKvTile;

  uint32_t qa[KS][4];
  {
    const bool va = row_a < p.T, vb = row_b < p.T;
    const __nv_bfloat16* qa_p = p.q + (size_t(min(row_a, p.T - 1)) * p.Hq + h) * HD;
    const __nv_bfloat16* qb_p = p.q + (size_t(min(row_b, p.T - 1)) * p.Hq + h) * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + t * 2;
      qa[ks][0] = va ? *reinterpret_cast<const uint32_t*>(qa_p + d) : 0u;
      qa[ks][1] = vb ? *reinterpret_cast<const uint32_t*>(qb_p + d) : 0u;
      qa[ks][2] = va ? *reinterpret_cast<const uint32_t*>(qa_p + d + 8) : 0u;
      qa[ks][3] = vb ? *reinterpret_cast<const uint32_t*>(qb_p + d + 8) : 0u;
    }
  }
  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  auto issue = [&](int tile, int stage) {   // whole block: 4 pages of K and of V
    char* kd = smem + stage * 2 * TILE_BYTES;
    char* vd = kd + TILE_BYTES;
    for (int idx = threadIdx.x; idx < 4 * kFpPage * CH; idx += kFpThreads) {
      const int pg = idx / (kFpPage * CH), rem = idx % (kFpPage * CH);
      const int r = rem / CH, c = rem % CH;
      const int page = tile * 4 + pg;
      if (page * kFpPage >= kv_end) continue;           // nothing cached there yet
      const int blk = p.block_table[page];
      const size_t src = (size_t(blk) * p.Hkv + kvh) * PAGE_BYTES + size_t(rem) * 16;
      const int off = pg * PAGE_BYTES + r * (HD * 2) + ((c ^ (r & 7)) << 4);
      fp_cp_async16(kd + off, reinterpret_cast<const char*>(p.k_cache) + src);
      fp_cp_async16(vd + off, reinterpret_cast<const char*>(p.v_cache) + src);
    }
  };

  if (tile_begin < tile_end) issue(tile_begin, 0);
  fp_commit();
  int stage = 0;
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    if (tile + 1 < tile_end) issue(tile + 1, stage ^ 1);
    fp_commit();
    fp_wait<1>();
    __syncthreads();
    const uint32_t kbase = smem_u32(smem + stage * 2 * TILE_BYTES);
    const uint32_t vbase = kbase + TILE_BYTES;
    // two pages (32 keys) per step: one running-max update and one rescale of the output
    // accumulators per 32 keys, and no mask arithmetic on steps that lie wholly below the diagonal
    const int warp_pos_lo = p.pos0 + q0 + warp * 16, warp_pos_hi = warp_pos_lo + 15;
#pragma unroll 1
    for (int pp = 0; pp < 2; ++pp) {
      const int key0 = tile * kFpKvTile + pp * 2 * kFpPage;
      // whole step above the diagonal for every row of this warp, or outside the cached range
      if (key0 > warp_pos_hi || key0 >= kv_end) break;
      if (p.window > 0 && key0 + 31 <= warp_pos_lo - p.window) continue;
      const bool second = key0 + kFpPage <= warp_pos_hi && key0 + kFpPage < kv_end;   // page 2 has visible keys
      const bool need_mask = key0 + 31 > warp_pos_lo || p.window > 0;
      float sv[2][8];
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        if (q2 == 0 || second) {
          const uint32_t kpage = kbase + (pp * 2 + q2) * PAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi >> 1) * 8 + r, c = 2 * ks + (mi & 1);
            uint32_t kb[4];
            fp_ldm4(kb, kpage + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
            fp_mma(s0, qa[ks], kb[0], kb[1]);
            fp_mma(s1, qa[ks], kb[2], kb[3]);
          }
        }
        // row a: keys kt, kt+1, kt+8, kt+9 ; row b: the same keys
        sv[q2][0] = s0[0]; sv[q2][1] = s0[1]; sv[q2][2] = s1[0]; sv[q2][3] = s1[1];
        sv[q2][4] = s0[2]; sv[q2][5] = s0[3]; sv[q2][6] = s1[2]; sv[q2][7] = s1[3];
      }
      if (need_mask || !second) {
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int kt = key0 + q2 * kFpPage + t * 2;
          const int keys[4] = {kt, kt + 1, kt + 8, kt + 9};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            bool oka = keys[i] <= pos_a && (q2 == 0 || second), okb = keys[i] <= pos_b && (q2 == 0 || second);
            if (p.window > 0) { oka = oka && keys[i] > pos_a - p.window; okb = okb && keys[i] > pos_b - p.window; }
            sv[q2][i] = oka ? sv[q2][i] * p.scale_log2 : -INFINITY;
            sv[q2][4 + i] = okb ? sv[q2][4 + i] * p.scale_log2 : -INFINITY;
          }
        }
      } else {
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
          for (int i = 0; i < 8; ++i) sv[q2][i] *= p.scale_log2;
      }
      float mx0 = fmaxf(fmaxf(fmaxf(sv[0][0], sv[0][1]), fmaxf(sv[0][2], sv[0][3])),
                        fmaxf(fmaxf(sv[1][0], sv[1][1]), fmaxf(sv[1][2], sv[1][3])));
      float mx1 = fmaxf(fmaxf(fmaxf(sv[0][4], sv[0][5]), fmaxf(sv[0][6], sv[0][7])),
                        fmaxf(fmaxf(sv[1][4], sv[1][5]), fmaxf(sv[1][6], sv[1][7])));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
      // a row may have no visible key in this step (fully masked): keep its state unchanged
      const float c0 = (nm0 == -INFINITY) ? 1.f : exp2f(m0 - nm0);
      const float c1 = (nm1 == -INFINITY) ? 1.f : exp2f(m1 - nm1);
      m0 = nm0; m1 = nm1;
      const float sub0 = (m0 == -INFINITY) ? 0.f : m0, sub1 = (m1 == -INFINITY) ? 0.f : m1;
      uint32_t pa[2][4];
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        float pr[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pr[i] = exp2f(sv[q2][i] - sub0);            // exp2(-inf) = 0 for masked entries
          pr[4 + i] = exp2f(sv[q2][4 + i] - sub1);
        }
        ps0 += (pr[0] + pr[1]) + (pr[2] + pr[3]);
        ps1 += (pr[4] + pr[5]) + (pr[6] + pr[7]);
        pa[q2][0] = pack_bf16(pr[0], pr[1]); pa[q2][1] = pack_bf16(pr[4], pr[5]);
        pa[q2][2] = pack_bf16(pr[2], pr[3]); pa[q2][3] = pack_bf16(pr[6], pr[7]);
      }
      l0 = l0 * c0 + ps0;
      l1 = l1 * c1 + ps1;
#pragma unroll
      for (int j = 0; j < NT; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        if (q2 == 0 || second) {
          const uint32_t vpage = vbase + (pp * 2 + q2) * PAGE_BYTES;
#pragma unroll
          for (int j = 0; j < NT; j += 2) {
            const int mi = lane >> 3, r = lane & 7;
            const int tok = (mi & 1) * 8 + r, c = j + (mi >> 1);
            uint32_t vb[4];
            fp_ldm4t(vb, vpage + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
            fp_mma(o[j], pa[q2], vb[0], vb[1]);
            fp_mma(o[j + 1], pa[q2], vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();          // everyone is done with this stage before it is refilled
    stage ^= 1;
  }
  fp_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d = j * 8 + t * 2;
    if (row_a < p.T)
      *reinterpret_cast<uint32_t*>(p.out + (size_t(row_a) * p.Hq + h) * HD + d) = pack_bf16(o[j][0] * i0, o[j][1] * i0);
    if (row_b < p.T)
      *reinterpret_cast<uint32_t*>(p.out + (size_t(row_b) * p.Hq + h) * HD + d) = pack_bf16(o[j][2] * i1, o[j][3] * i1);
  }
  pdl_launch_dependents();
}

}  // namespace rb

using namespace rb;

// q, out: [T, Hq, HD] bf16; caches [blocks, Hkv, 16, HD]; block_table: the sequence's row (int32);
// queries are at positions pos0 .. pos0+T-1 and the cache already holds keys 0 .. pos0+T-1.
extern "C" int rmlx_flash_prefill_paged(const void* q, const void* k_cache, const void* v_cache,
                                        const int* block_table, void* out, int T, int Hq, int Hkv,
                                        int HD, int pos0, int window, float scale, int pdl,
                                        cudaStream_t st) {
  if (T < 1 || Hq % Hkv || pos0 < 0) return -2;
  FpParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_table = block_table; p.out = static_cast<__nv_bfloat16*>(out);
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.pos0 = pos0; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((T + 63) / 64, Hq);
  if (HD == 128) {
    const size_t smem = 2 * 2 * 4 * kFpPage * 128 * 2;   // 64 KB
    auto kern = flash_prefill_kernel<128>;
    RB_CHECK(set_max_smem(kern, smem));
    return launch(kern, grid, dim3(kFpThreads), smem, st, pdl != 0, p);
  }
  if (HD == 64) {
    const size_t smem = 2 * 2 * 4 * kFpPage * 64 * 2;    // 32 KB
    auto kern = flash_prefill_kernel<64>;
    RB_CHECK(set_max_smem(kern, smem));
    return launch(kern, grid, dim3(kFpThreads), smem, st, pdl != 0, p);
  }
  return -2;
}
