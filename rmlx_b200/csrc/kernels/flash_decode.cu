// Paged flash-decode attention (one new query token per sequence) for grouped-query attention.
//
// A block owns one (sequence, kv-head, 16-query-head tile, KV split). The 16 query heads that
// share a kv head form the M=16 side of m16n8k16 tensor-core tiles, so K and V pages are read
// once per kv head, not once per query head. Four warps walk the split's pages (16 tokens each,
// located through the block table) with a two-stage cp.async pipeline into swizzled shared memory;
// each warp keeps its own online-softmax state, the block merges them, and when the context was
// split across blocks the last block to finish merges the partial results, all in one launch.
//
// The tensor-core path here is mma.sync on purpose: the useful M is 16 rows and the kernel is
// bound by KV bytes and latency; a tcgen05 tile (M >= 64, TMEM round trip) has nothing to gain.
//
// Replaces sdpa_decode_batched_* over contiguous slabs (crates/rmlx-core/src/ops/sdpa.rs:810,1541)
// and the CPU page gather of PagedKvCache::get_keys (crates/rmlx-nn/src/paged_kv_cache.rs:479-547).
//
// Cache layout: [num_blocks, kv_heads, page=16, head_dim] bf16 for K and for V.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kPage = 16;
constexpr int kFdWarps = 4;
constexpr int kFdThreads = kFdWarps * 32;
constexpr int kFdMaxSplits = 64;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct FdParams {
  const __nv_bfloat16* q;        // [B, Hq, HD]
  const __nv_bfloat16* k_cache;  // [blocks, Hkv, 16, HD]  (8-bit cache: uint8 of the same shape)
  const __nv_bfloat16* v_cache;
  const char* k_sb;              // 8-bit cache: [blocks, Hkv, 16, HD/64] (scale, bias) bf16 pairs
  const char* v_sb;
  const int* block_table;        // [B, max_blocks]
  const int* seq_lens;           // [B] tokens in the cache including the current one
  __nv_bfloat16* out;            // [B, Hq, HD]
  float* part_o;                 // [B, Hkv*gtiles, S, 16, HD]
  float* part_ml;                // [B, Hkv*gtiles, S, 16, 2]
  unsigned int* tickets;         // [B * Hkv*gtiles], zero on entry, zero on exit
  int max_blocks, Hq, Hkv, G, gtiles, S, window;
  float scale_log2;              // softmax scale * log2(e)
};

// KVQ: the cache holds 8-bit affine values (x = q * scale + bias per token and group of 64 along
// the head dimension; crates/rmlx-nn/src/attention.rs:4438-4680 keeps the same format on the host).
// A stage then holds the raw pages and their (scale, bias) pairs, and the warp expands a page into
// its own bf16 tile (same swizzled layout) right before it multiplies: half the DRAM bytes per
// token, the tensor-core part unchanged.
template <int HD, int NST, bool KVQ = false>
__global__ void __launch_bounds__(kFdThreads) flash_decode_kernel(FdParams p) {
  constexpr int CH = HD / 8;             // 16-byte chunks per row
  constexpr int KS = HD / 16;            // k-steps of the QK^T product
  constexpr int NT = HD / 8;             // n-tiles of the PV product
  constexpr int PAGE_BYTES = kPage * HD * 2;
  constexpr int G64 = HD / 64;                    // quantisation groups per row
  constexpr int RAW_PAGE = kPage * HD;            // bytes of an 8-bit page
  constexpr int SB_PAGE = kPage * G64 * 4;        // bytes of a page's (scale, bias) pairs
  constexpr int STAGE_BYTES = KVQ ? 2 * RAW_PAGE + 2 * SB_PAGE : 2 * PAGE_BYTES;
  constexpr int WARP_BYTES = NST * STAGE_BYTES + (KVQ ? 2 * PAGE_BYTES : 0);
  extern __shared__ __align__(128) char smem[];
  // per warp: NST stages x (K page, V page) (+ one expanded K/V tile for the 8-bit cache); reused
  // afterwards for the cross-warp merge
  char* wsm = smem + (threadIdx.x >> 5) * WARP_BYTES;
  __shared__ float s_m[kFdWarps][16], s_l[kFdWarps][16];
  __shared__ unsigned int s_last;

  const int split = blockIdx.x, yt = blockIdx.y, b = blockIdx.z;
  const int kvh = yt / p.gtiles, gt = yt % p.gtiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const int len = p.seq_lens[b];
  const int first = (p.window > 0 && len > p.window) ? len - p.window : 0;  // first visible token
  const int pg_begin = first / kPage;
  const int pg_total = (len + kPage - 1) / kPage - pg_begin;
  const int pg_per_split = (pg_total + p.S - 1) / p.S;
  const int pg0 = pg_begin + split * pg_per_split;
  const int pg1 = min(pg0 + pg_per_split, pg_begin + pg_total);

  // Q fragments (rows = query heads of this tile; rows beyond G are zero).
  uint32_t qa[KS][4];
  {
    const int h0 = gt * 16 + g, h1 = h0 + 8;
    const __nv_bfloat16* q0 = p.q + (size_t(b) * p.Hq + size_t(kvh) * p.G + h0) * HD;
    const __nv_bfloat16* q1 = p.q + (size_t(b) * p.Hq + size_t(kvh) * p.G + h1) * HD;
    const bool v0 = h0 < p.G, v1 = h1 < p.G;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int d = ks * 16 + t * 2;
      qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
      qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
      qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
      qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
    }
  }

  float o[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int* bt = p.block_table + size_t(b) * p.max_blocks;
  auto issue = [&](int pg, int stage) {
    const int blk = RB_BOUNDS(pg, p.max_blocks) ? bt[pg] : 0;   // page 0 is the reserved page
    if (KVQ) {
      const size_t pgi = size_t(blk) * p.Hkv + kvh;
      const char* ksrc = reinterpret_cast<const char*>(p.k_cache) + pgi * RAW_PAGE;
      const char* vsrc = reinterpret_cast<const char*>(p.v_cache) + pgi * RAW_PAGE;
      char* kd = wsm + stage * STAGE_BYTES;
      char* vd = kd + RAW_PAGE;
#pragma unroll
      for (int i = 0; i < (RAW_PAGE / 16) / 32; ++i) {
        const int idx = i * 32 + lane;
        cp_async16(kd + idx * 16, ksrc + idx * 16);
        cp_async16(vd + idx * 16, vsrc + idx * 16);
      }
      if (lane < SB_PAGE / 16) {
        cp_async16(vd + RAW_PAGE + lane * 16, p.k_sb + pgi * SB_PAGE + lane * 16);
        cp_async16(vd + RAW_PAGE + SB_PAGE + lane * 16, p.v_sb + pgi * SB_PAGE + lane * 16);
      }
      return;
    }
    const char* ksrc = reinterpret_cast<const char*>(p.k_cache) +
                       (size_t(blk) * p.Hkv + kvh) * PAGE_BYTES;
    const char* vsrc = reinterpret_cast<const char*>(p.v_cache) +
                       (size_t(blk) * p.Hkv + kvh) * PAGE_BYTES;
    char* kd = wsm + stage * 2 * PAGE_BYTES;
    char* vd = kd + PAGE_BYTES;
#pragma unroll
    for (int i = 0; i < (kPage * CH) / 32; ++i) {
      const int idx = i * 32 + lane;       // chunk index inside the page
      const int r = idx / CH, c = idx % CH;
      const int off = r * (HD * 2) + ((c ^ (r & 7)) << 4);
      cp_async16(kd + off, ksrc + idx * 16);
      cp_async16(vd + off, vsrc + idx * 16);
    }
  };

  // 8-bit cache: expand stage `stage` (raw K and V pages) into the warp's bf16 tile pair.
  auto expand = [&](int stage) {
    const char* raw = wsm + stage * STAGE_BYTES;
    char* tile = wsm + NST * STAGE_BYTES;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const char* src = raw + which * RAW_PAGE;
      const char* sb = raw + 2 * RAW_PAGE + which * SB_PAGE;
      char* dst = tile + which * PAGE_BYTES;
#pragma unroll
      for (int i = 0; i < (RAW_PAGE / 16) / 32; ++i) {
        const int idx = i * 32 + lane;
        const int r = idx / (HD / 16), k = idx % (HD / 16);     // token, 16-value piece
        const uint4 w = *reinterpret_cast<const uint4*>(src + idx * 16);
        const uint32_t sbv = *reinterpret_cast<const uint32_t*>(sb + (r * G64 + (k >> 2)) * 4);
        const float sc = __uint_as_float(sbv << 16), bi = __uint_as_float(sbv & 0xffff0000u);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float f0 = fmaf(float(ww[j] & 0xffu), sc, bi), f1 = fmaf(float((ww[j] >> 8) & 0xffu), sc, bi);
          const float f2 = fmaf(float((ww[j] >> 16) & 0xffu), sc, bi), f3 = fmaf(float(ww[j] >> 24), sc, bi);
          o[2 * j] = pack_bf16(f0, f1);
          o[2 * j + 1] = pack_bf16(f2, f3);
        }
        char* row = dst + r * (HD * 2);
        *reinterpret_cast<uint4*>(row + (((2 * k) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4*>(row + (((2 * k + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  };

  // Ring of NST stages per warp: the first NST pages are requested up front, so their DRAM
  // latencies overlap instead of adding up; a stage is refilled as soon as it has been consumed.
  int pg = pg0 + warp;
#pragma unroll
  for (int s = 0; s < NST; ++s) {
    if (pg + s * kFdWarps < pg1) issue(pg + s * kFdWarps, s);
    cp_async_commit();
  }
  int stage = 0;
  for (; pg < pg1; pg += kFdWarps) {
    cp_async_wait<NST - 1>();
    __syncwarp();
    if (KVQ) { expand(stage); __syncwarp(); }
    const uint32_t kbase = smem_u32(KVQ ? wsm + NST * STAGE_BYTES : wsm + stage * 2 * PAGE_BYTES);
    const uint32_t vbase = kbase + PAGE_BYTES;

    // S = Q K^T for 16 tokens: two n-tiles of 8 tokens.
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = (mi >> 1) * 8 + r, c = 2 * ks + (mi & 1);
      uint32_t kb[4];
      ldmatrix_x4(kb, kbase + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
      mma_bf16_16816(s0, qa[ks], kb[0], kb[1]);
      mma_bf16_16816(s1, qa[ks], kb[2], kb[3]);
    }
    // scale, mask tokens outside [first, len)
    const int tok0 = pg * kPage + t * 2;
    float sv[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};
    const int tk[4] = {tok0, tok0 + 1, tok0 + 8, tok0 + 9};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = tk[i] < len && tk[i] >= first;
      sv[i] = ok ? sv[i] * p.scale_log2 : -INFINITY;
      sv[4 + i] = ok ? sv[4 + i] * p.scale_log2 : -INFINITY;
    }
    float mx0 = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    float mx1 = fmaxf(fmaxf(sv[4], sv[5]), fmaxf(sv[6], sv[7]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
    // a page always holds at least one visible token, so nm is finite here
    const float c0 = exp2f(m0 - nm0), c1 = exp2f(m1 - nm1);
    m0 = nm0; m1 = nm1;
    float pr[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) { pr[i] = exp2f(sv[i] - m0); pr[4 + i] = exp2f(sv[4 + i] - m1); }
    l0 = l0 * c0 + (pr[0] + pr[1] + pr[2] + pr[3]);
    l1 = l1 * c1 + (pr[4] + pr[5] + pr[6] + pr[7]);
    uint32_t pa[4] = {pack_bf16(pr[0], pr[1]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[2], pr[3]),
                      pack_bf16(pr[6], pr[7])};
#pragma unroll
    for (int j = 0; j < NT; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    // O += P V : V fragments through transposing ldmatrix, two n-tiles per load.
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = (mi & 1) * 8 + r, c = j + (mi >> 1);
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, vbase + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
      mma_bf16_16816(o[j], pa, vb[0], vb[1]);
      mma_bf16_16816(o[j + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();
    if (pg + NST * kFdWarps < pg1) issue(pg + NST * kFdWarps, stage);
    cp_async_commit();
    stage = (stage + 1 == NST) ? 0 : stage + 1;
  }
  cp_async_wait<0>();
  // row sums live in the quad: finish them
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the four warps of the block ----
  __syncthreads();  // everyone is done with the staging buffers
  float* so = reinterpret_cast<float*>(smem);  // [warp][16][HD]
  if (t == 0) { s_m[warp][g] = m0; s_m[warp][g + 8] = m1; s_l[warp][g] = l0; s_l[warp][g + 8] = l1; }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d = j * 8 + t * 2;
    *reinterpret_cast<float2*>(so + (warp * 16 + g) * HD + d) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2*>(so + (warp * 16 + g + 8) * HD + d) = make_float2(o[j][2], o[j][3]);
  }
  __syncthreads();
  const size_t tile = (size_t(b) * p.Hkv * p.gtiles + yt);
  for (int idx = threadIdx.x; idx < 16 * HD; idx += kFdThreads) {
    const int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kFdWarps; ++w) M = fmaxf(M, s_m[w][row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kFdWarps; ++w) {
      const float f = (s_m[w][row] == -INFINITY) ? 0.f : exp2f(s_m[w][row] - M);
      L += s_l[w][row] * f;
      acc += so[(w * 16 + row) * HD + d] * f;
    }
    const int h = gt * 16 + row;
    if (p.S == 1) {
      if (h < p.G)
        p.out[(size_t(b) * p.Hq + size_t(kvh) * p.G + h) * HD + d] =
            __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      p.part_o[((tile * p.S + split) * 16 + row) * HD + d] = acc;
      if (d == 0) {
        p.part_ml[((tile * p.S + split) * 16 + row) * 2] = M;
        p.part_ml[((tile * p.S + split) * 16 + row) * 2 + 1] = L;
      }
    }
  }
  if (p.S == 1) { pdl_launch_dependents(); return; }

  // ---- last block of this tile merges the splits ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.tickets + tile, 1u) == unsigned(p.S - 1)) ? 1u : 0u;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Per-split weights exp2(m_s - M) / L for the 16 rows go to shared memory first (one parallel
  // pass over the small (max, sum) table); the big pass over the partial outputs then has no
  // dependent loads and runs eight splits at a time.
  float* wgt = reinterpret_cast<float*>(smem);        // [S][16]
  float* mls = wgt + kFdMaxSplits * 16;               // [S][16][2] copy of the (max, sum) table
  __syncthreads();
  for (int i = threadIdx.x; i < p.S * 32; i += kFdThreads) mls[i] = p.part_ml[tile * p.S * 32 + i];
  __syncthreads();
  if (threadIdx.x < 16) {
    const int row = threadIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < p.S; ++s) M = fmaxf(M, mls[s * 32 + row * 2]);
    float L = 0.f;
    for (int s = 0; s < p.S; ++s) {
      const float ms = mls[s * 32 + row * 2];
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      wgt[s * 16 + row] = f;
      L += mls[s * 32 + row * 2 + 1] * f;
    }
    const float invL = L > 0.f ? 1.f / L : 0.f;
    for (int s = 0; s < p.S; ++s) wgt[s * 16 + row] *= invL;
  }
  __syncthreads();
  // Each thread owns four consecutive d of one row at a time and keeps sixteen 16-byte loads in
  // flight: the partials sit in L2, so the merge is a latency problem, not a bandwidth one.
  const float4* po4 = reinterpret_cast<const float4*>(p.part_o + tile * p.S * 16 * HD);
  constexpr int D4 = HD / 4;
  for (int idx = threadIdx.x; idx < 16 * D4; idx += kFdThreads) {
    const int row = idx / D4, d4 = idx % D4;
    const int h = gt * 16 + row;
    if (h >= p.G) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < p.S; s += 16) {
      float4 v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j)
        v[j] = (s + j < p.S) ? po4[(size_t(s + j) * 16 + row) * D4 + d4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float w = (s + j < p.S) ? wgt[(s + j) * 16 + row] : 0.f;
        acc.x = fmaf(v[j].x, w, acc.x); acc.y = fmaf(v[j].y, w, acc.y);
        acc.z = fmaf(v[j].z, w, acc.z); acc.w = fmaf(v[j].w, w, acc.w);
      }
    }
    uint2 o;
    o.x = pack_bf16(acc.x, acc.y);
    o.y = pack_bf16(acc.z, acc.w);
    *reinterpret_cast<uint2*>(p.out + (size_t(b) * p.Hq + size_t(kvh) * p.G + h) * HD + d4 * 4) = o;
  }
  if (threadIdx.x == 0) p.tickets[tile] = 0u;
  pdl_launch_dependents();
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("flash_decode.cu")


// Scratch sizes for a launch with the given shape (floats / uint32 counts).
extern "C" int rmlx_flash_decode_gtiles(int Hq, int Hkv) { return ((Hq / Hkv) + 15) / 16; }
extern "C" long long rmlx_flash_decode_part_o_elems(int B, int Hq, int Hkv, int S, int HD) {
  return 1LL * B * Hkv * rmlx_flash_decode_gtiles(Hq, Hkv) * S * 16 * HD;
}
extern "C" long long rmlx_flash_decode_part_ml_elems(int B, int Hq, int Hkv, int S) {
  return 1LL * B * Hkv * rmlx_flash_decode_gtiles(Hq, Hkv) * S * 16 * 2;
}
extern "C" long long rmlx_flash_decode_ticket_elems(int B, int Hq, int Hkv) {
  return 1LL * B * Hkv * rmlx_flash_decode_gtiles(Hq, Hkv);
}

// `splits` in [1, 64]: how many blocks share one sequence's context. `tickets` must be zero on the
// first call; the kernel leaves it zero. `window` > 0 restricts attention to the last `window`
// tokens (sliding-window models). head_dim 64 or 128, page size 16.
static int fd_launch(const void* q, const void* k_cache, const void* v_cache, const void* k_sb,
                     const void* v_sb, const int* block_table, const int* seq_lens, void* out,
                     float* part_o, float* part_ml, unsigned int* tickets, int B, int Hq, int Hkv,
                     int HD, int max_blocks, int splits, int window, float scale, int pdl,
                     cudaStream_t st) {
  if (B < 1 || Hq % Hkv || splits < 1 || splits > kFdMaxSplits) return -2;
  if (splits > 1 && (!part_o || !part_ml || !tickets)) return -2;
  const bool kvq = k_sb != nullptr;
  FdParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.k_sb = static_cast<const char*>(k_sb); p.v_sb = static_cast<const char*>(v_sb);
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml; p.tickets = tickets;
  p.max_blocks = max_blocks; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv;
  p.gtiles = rmlx_flash_decode_gtiles(Hq, Hkv); p.S = splits; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(splits, Hkv * p.gtiles, B);
  // Few blocks (small batch): deep per-warp ring, one block per SM. Many blocks: shallow ring so
  // several blocks share an SM. Either way the staging area (>= 32 KB at HD 128, 16 KB at HD 64)
  // covers the cross-warp merge buffer and the split-merge tables.
  const bool deep = size_t(splits) * Hkv * p.gtiles * B <= size_t(2 * sm_count());
#define RB_FD(HD_, NST_, KVQ_)                                                                    \
  {                                                                                               \
    const size_t stage = KVQ_ ? 2 * kPage * HD_ + 2 * kPage * (HD_ / 64) * 4 : 2 * kPage * HD_ * 2; \
    const size_t smem = size_t(kFdWarps) * (NST_ * stage + (KVQ_ ? 2 * kPage * HD_ * 2 : 0));     \
    auto kern = flash_decode_kernel<HD_, NST_, KVQ_>;                                             \
    RB_CHECK(set_max_smem(kern, smem));                                                           \
    return launch(kern, grid, dim3(kFdThreads), smem, st, pdl != 0, p);                           \
  }
  if (kvq) {
    if (HD == 128) { if (deep) RB_FD(128, 4, true) else RB_FD(128, 2, true) }
    if (HD == 64) { if (deep) RB_FD(64, 4, true) else RB_FD(64, 2, true) }
    return -2;
  }
  if (HD == 128) { if (deep) RB_FD(128, 4, false) else RB_FD(128, 2, false) }
  if (HD == 64) { if (deep) RB_FD(64, 4, false) else RB_FD(64, 2, false) }
#undef RB_FD
  return -2;
}

extern "C" int rmlx_flash_decode_paged(const void* q, const void* k_cache, const void* v_cache,
                                       const int* block_table, const int* seq_lens, void* out,
                                       float* part_o, float* part_ml, unsigned int* tickets, int B,
                                       int Hq, int Hkv, int HD, int max_blocks, int splits,
                                       int window, float scale, int pdl, cudaStream_t st) {
  return fd_launch(q, k_cache, v_cache, nullptr, nullptr, block_table, seq_lens, out, part_o, part_ml,
                   tickets, B, Hq, Hkv, HD, max_blocks, splits, window, scale, pdl, st);
}

// The same attention over an 8-bit cache: k_q / v_q uint8 [blocks, Hkv, 16, HD], k_sb / v_sb bf16
// [blocks, Hkv, 16, HD/64, 2] (scale, bias), as written by rmlx_rope_kv_write_q8 (kv_q8.cu).
extern "C" int rmlx_flash_decode_paged_q8(const void* q, const void* k_q, const void* k_sb,
                                          const void* v_q, const void* v_sb, const int* block_table,
                                          const int* seq_lens, void* out, float* part_o,
                                          float* part_ml, unsigned int* tickets, int B, int Hq,
                                          int Hkv, int HD, int max_blocks, int splits, int window,
                                          float scale, int pdl, cudaStream_t st) {
  if (!k_sb || !v_sb) return -2;
  return fd_launch(q, k_q, v_q, k_sb, v_sb, block_table, seq_lens, out, part_o, part_ml, tickets, B,
                   Hq, Hkv, HD, max_blocks, splits, window, scale, pdl, st);
}

// ------------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in flash_decode_noalloc.h). Some users of this
// library cannot call the CUDA allocator where they run attention: an engine that pre-partitions
// all device memory, a latency-critical loop that must not block on allocator locks, a plug-in
// API that passes only inputs and outputs. For them the split-KV scratch lives in this file-scope
// device array. In host code the array's name is only a host-side handle, not a device address,
// so the address is looked up once per device with cudaGetSymbolAddress and that pointer is what
// the kernel receives.
// ------------------------------------------------------------------------------------------------
#include "flash_decode_noalloc.h"

namespace {
constexpr size_t kNaPartO = size_t(RMLX_FD_NOALLOC_MAX_TILES) * RMLX_FD_NOALLOC_MAX_SPLITS * 16 *
                            RMLX_FD_NOALLOC_MAX_HEAD_DIM;                       // floats
constexpr size_t kNaPartMl = size_t(RMLX_FD_NOALLOC_MAX_TILES) * RMLX_FD_NOALLOC_MAX_SPLITS * 16 * 2;
constexpr size_t kNaTickets = RMLX_FD_NOALLOC_MAX_TILES;                        // uint32
constexpr size_t kNaBytes = (kNaPartO + kNaPartMl) * sizeof(float) + kNaTickets * sizeof(unsigned int);

static __device__ __align__(256) unsigned char g_fd_noalloc_scratch[kNaBytes];

constexpr int kNaMaxDevices = 64;
void* g_fd_noalloc_ptr[kNaMaxDevices] = {nullptr};
}  // namespace

extern "C" const char* rmlx_flash_decode_noalloc_error(int code) {
  switch (code) {
    case RMLX_FD_NOALLOC_TOO_LARGE:
      return "flash_decode_paged_noalloc: batch*kv_heads*head_tiles > 64, splits > 16 or head_dim > 128 "
             "exceeds the built-in scratch; use rmlx_flash_decode_paged with caller-provided scratch";
    case RMLX_FD_NOALLOC_SETUP_FAILED:
      return "flash_decode_paged_noalloc: could not resolve the device address of the built-in scratch";
    default:
      return nullptr;
  }
}

extern "C" int rmlx_flash_decode_paged_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                               const int* block_table, const int* seq_lens, void* out,
                                               int B, int Hq, int Hkv, int HD, int max_blocks,
                                               int splits, int window, float scale,
                                               cudaStream_t stream) {
  if (B < 1 || Hkv < 1 || Hq < 1 || Hq % Hkv || splits < 1) return -2;
  const long long tiles = 1LL * B * Hkv * rmlx_flash_decode_gtiles(Hq, Hkv);
  if (tiles > RMLX_FD_NOALLOC_MAX_TILES || splits > RMLX_FD_NOALLOC_MAX_SPLITS ||
      HD > RMLX_FD_NOALLOC_MAX_HEAD_DIM)
    return RMLX_FD_NOALLOC_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNaMaxDevices)
    return RMLX_FD_NOALLOC_SETUP_FAILED;
  if (g_fd_noalloc_ptr[dev] == nullptr) {
    // once per device, with that device current; not inside a stream capture
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fd_noalloc_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return RMLX_FD_NOALLOC_SETUP_FAILED;
    }
    g_fd_noalloc_ptr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_fd_noalloc_ptr[dev]);
  float* part_o = reinterpret_cast<float*>(base);
  float* part_ml = part_o + kNaPartO;
  unsigned int* tickets = reinterpret_cast<unsigned int*>(part_ml + kNaPartMl);
  // the tickets are the only part that must start at zero; the partials are fully rewritten
  RB_CHECK(cudaMemsetAsync(tickets, 0, kNaTickets * sizeof(unsigned int), stream));
  return rmlx_flash_decode_paged(q, k_cache, v_cache, block_table, seq_lens, out, part_o, part_ml,
                                 tickets, B, Hq, Hkv, HD, max_blocks, splits, window, scale, 0, stream);
}
