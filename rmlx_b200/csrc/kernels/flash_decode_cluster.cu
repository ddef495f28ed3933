// Paged split-KV flash decode for SMALL batches, where one sequence has to fill the machine:
// the context of a (sequence, kv-head, 16-query-head tile) is cut into many splits (one block
// each, 8 warps, about one page of 16 tokens per warp), and the splits are merged in two levels
// without a serial tail:
//   1. the 8 blocks of a thread-block CLUSTER merge through distributed shared memory: after a
//      cluster barrier block r reads head-dim columns [r*HD/8, (r+1)*HD/8) of all 8 partial
//      outputs straight out of its neighbours' shared memory;
//   2. when a tile spans several clusters each writes one partial per cluster, and the last
//      cluster to arrive (a ticket per tile) merges those few partials, again column-sliced over
//      its 8 blocks.
// With the 64 q / 4 kv head model at context 4096 this is 128 blocks (4 tiles x 4 clusters x 8)
// instead of 64 blocks and a last-block pass over 16 partials; with one kv head per rank (TP 8)
// it is 144 blocks instead of 16.
//
// The per-warp page loop (cp.async ring into swizzled shared memory, mma.sync m16n8k16 with the
// 16 query heads of a kv head as M) is the one of flash_decode.cu. M is 16 rows and the kernel is
// bound by latency, so mma.sync is the tensor-core path on purpose.
//
// Replaces sdpa_decode_batched_* over contiguous slabs (crates/rmlx-core/src/ops/sdpa.rs:810,1541).
#include <cooperative_groups.h>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace cg = cooperative_groups;

namespace rb {

constexpr int kFcPage = 16;
constexpr int kFcWarps = 8;
constexpr int kFcThreads = kFcWarps * 32;
constexpr int kFcMaxCluster = 16;
constexpr int kFcMaxClusters = 32;     // clusters per tile

__device__ __forceinline__ void fc_cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void fc_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fc_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fc_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fc_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fc_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct FcParams {
  const __nv_bfloat16* q;        // [B, Hq, HD]
  const __nv_bfloat16* k_cache;  // [blocks, Hkv, 16, HD]
  const __nv_bfloat16* v_cache;
  const int* block_table;        // [B, max_blocks]
  const int* seq_lens;           // [B] tokens in the cache including the current one
  __nv_bfloat16* out;            // [B, Hq, HD]
  float* part_o;                 // [tiles, NC, 16, HD]   (NC > 1 only)
  float* part_ml;                // [tiles, NC, 16, 2]
  unsigned int* tickets;         // [tiles], zero on entry, zero on exit
  int max_blocks, Hq, Hkv, G, gtiles, NC, window;
  float scale_log2;              // softmax scale * log2(e)
};

// Shared memory: per warp 2 stages x (K page, V page), reused as [warp][16][HD] fp32 for the
// block merge; then the block's merged partial [16][HD] fp32 + (m, l)[16] that its cluster
// neighbours read.
template <int HD, int kFcCluster>
__global__ void __launch_bounds__(kFcThreads) flash_decode_cluster_kernel(FcParams p) {
  constexpr int CH = HD / 8;             // 16-byte chunks per row
  constexpr int KS = HD / 16;            // k-steps of the QK^T product
  constexpr int NT = HD / 8;             // n-tiles of the PV product
  constexpr int PAGE_BYTES = kFcPage * HD * 2;
  constexpr int NST = 2;
  constexpr int COLS = HD / kFcCluster;  // head-dim columns this block merges
  extern __shared__ __align__(128) char smem[];
  char* wsm = smem + (threadIdx.x >> 5) * (NST * 2 * PAGE_BYTES);
  float* blk_o = reinterpret_cast<float*>(smem + kFcWarps * NST * 2 * PAGE_BYTES);   // [16][HD]
  float* blk_ml = blk_o + 16 * HD;                                                    // [16][2]
  __shared__ float s_m[kFcWarps][16], s_l[kFcWarps][16];
  __shared__ float s_w[kFcMaxClusters][16];
  __shared__ unsigned int s_last;

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned crank = cluster.block_rank();
  const int split = blockIdx.x, S = gridDim.x, yt = blockIdx.y, b = blockIdx.z;
  const int cl = split / kFcCluster;     // this cluster's index inside the tile
  const int kvh = yt / p.gtiles, gt = yt % p.gtiles;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  pdl_launch_dependents();
  pdl_wait();
  const int len = p.seq_lens[b];
  const int first = (p.window > 0 && len > p.window) ? len - p.window : 0;  // first visible token
  const int pg_begin = first / kFcPage;
  const int pg_total = (len + kFcPage - 1) / kFcPage - pg_begin;
  const int pg_per_split = (pg_total + S - 1) / S;
  const int pg0 = pg_begin + split * pg_per_split;
  const int pg1 = min(pg0 + pg_per_split, pg_begin + pg_total);

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
    const char* ksrc = reinterpret_cast<const char*>(p.k_cache) + (size_t(blk) * p.Hkv + kvh) * PAGE_BYTES;
    const char* vsrc = reinterpret_cast<const char*>(p.v_cache) + (size_t(blk) * p.Hkv + kvh) * PAGE_BYTES;
    char* kd = wsm + stage * 2 * PAGE_BYTES;
    char* vd = kd + PAGE_BYTES;
#pragma unroll
    for (int i = 0; i < (kFcPage * CH) / 32; ++i) {
      const int idx = i * 32 + lane;
      const int r = idx / CH, c = idx % CH;
      const int off = r * (HD * 2) + ((c ^ (r & 7)) << 4);
      fc_cp_async16(kd + off, ksrc + idx * 16);
      fc_cp_async16(vd + off, vsrc + idx * 16);
    }
  };
  int pg = pg0 + warp;
#pragma unroll
  for (int s = 0; s < NST; ++s) {
    if (pg + s * kFcWarps < pg1) issue(pg + s * kFcWarps, s);
    fc_cp_async_commit();
  }
  int stage = 0;
  for (; pg < pg1; pg += kFcWarps) {
    fc_cp_async_wait<NST - 1>();
    __syncwarp();
    const uint32_t kbase = smem_u32(wsm + stage * 2 * PAGE_BYTES);
    const uint32_t vbase = kbase + PAGE_BYTES;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = (mi >> 1) * 8 + r, c = 2 * ks + (mi & 1);
      uint32_t kb[4];
      fc_ldmatrix_x4(kb, kbase + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
      fc_mma(s0, qa[ks], kb[0], kb[1]);
      fc_mma(s1, qa[ks], kb[2], kb[3]);
    }
    const int tok0 = pg * kFcPage + t * 2;
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
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      const int mi = lane >> 3, r = lane & 7;
      const int tok = (mi & 1) * 8 + r, c = j + (mi >> 1);
      uint32_t vb[4];
      fc_ldmatrix_x4_trans(vb, vbase + tok * (HD * 2) + ((c ^ (tok & 7)) << 4));
      fc_mma(o[j], pa, vb[0], vb[1]);
      fc_mma(o[j + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();
    if (pg + NST * kFcWarps < pg1) issue(pg + NST * kFcWarps, stage);
    fc_cp_async_commit();
    stage = (stage + 1 == NST) ? 0 : stage + 1;
  }
  fc_cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // ---- merge the eight warps of the block into blk_o / blk_ml ----
  __syncthreads();
  float* so = reinterpret_cast<float*>(smem);  // [warp][16][HD]
  if (t == 0) { s_m[warp][g] = m0; s_m[warp][g + 8] = m1; s_l[warp][g] = l0; s_l[warp][g + 8] = l1; }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d = j * 8 + t * 2;
    *reinterpret_cast<float2*>(so + (warp * 16 + g) * HD + d) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2*>(so + (warp * 16 + g + 8) * HD + d) = make_float2(o[j][2], o[j][3]);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * HD; idx += kFcThreads) {
    const int row = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kFcWarps; ++w) M = fmaxf(M, s_m[w][row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kFcWarps; ++w) {
      const float f = (s_m[w][row] == -INFINITY) ? 0.f : exp2f(s_m[w][row] - M);
      L += s_l[w][row] * f;
      acc += so[(w * 16 + row) * HD + d] * f;
    }
    blk_o[row * HD + d] = acc;
    if (d == 0) { blk_ml[row * 2] = M; blk_ml[row * 2 + 1] = L; }
  }
  cluster.sync();     // every block's partial is in its shared memory

  // ---- level 1: this block merges its column slice over the cluster's 8 partials (DSMEM) ----
  if (threadIdx.x < 16) {
    const int row = threadIdx.x;
    float ms[kFcCluster], ls[kFcCluster], M = -INFINITY;
#pragma unroll
    for (int r = 0; r < kFcCluster; ++r) {
      const float* rml = cluster.map_shared_rank(blk_ml, r);
      ms[r] = rml[row * 2]; ls[r] = rml[row * 2 + 1];
      M = fmaxf(M, ms[r]);
    }
    float L = 0.f;
#pragma unroll
    for (int r = 0; r < kFcCluster; ++r) {
      const float f = (ms[r] == -INFINITY) ? 0.f : exp2f(ms[r] - M);
      s_w[r][row] = f;
      L += ls[r] * f;
    }
    s_m[0][row] = M; s_l[0][row] = L;     // cluster-level (max, sum) of the row
  }
  __syncthreads();
  const size_t tile = size_t(b) * p.Hkv * p.gtiles + yt;
  const int c0 = int(crank) * COLS;
  float cacc = 0.f;                       // thread (row, col) of the slice: 16 x COLS <= 256 threads
  const int mrow = threadIdx.x / COLS, mcol = threadIdx.x % COLS;
  const bool mine = threadIdx.x < 16 * COLS;
  if (mine) {
#pragma unroll
    for (int r = 0; r < kFcCluster; ++r) {
      const float* ro = cluster.map_shared_rank(blk_o, r);
      cacc += ro[mrow * HD + c0 + mcol] * s_w[r][mrow];
    }
  }
  if (p.NC == 1) {
    if (mine) {
      const int h = gt * 16 + mrow;
      const float L = s_l[0][mrow];
      if (h < p.G)
        p.out[(size_t(b) * p.Hq + size_t(kvh) * p.G + h) * HD + c0 + mcol] =
            __float2bfloat16_rn(L > 0.f ? cacc / L : 0.f);
    }
    cluster.sync();   // nobody leaves while a neighbour still reads its shared memory
    return;
  }
  if (mine) p.part_o[((tile * p.NC + cl) * 16 + mrow) * HD + c0 + mcol] = cacc;
  if (crank == 0 && threadIdx.x < 16) {
    p.part_ml[((tile * p.NC + cl) * 16 + threadIdx.x) * 2] = s_m[0][threadIdx.x];
    p.part_ml[((tile * p.NC + cl) * 16 + threadIdx.x) * 2 + 1] = s_l[0][threadIdx.x];
  }
  __threadfence();
  cluster.sync();     // the cluster's partial is complete and visible; DSMEM reads are done
  if (crank == 0 && threadIdx.x == 0)
    s_last = (atomicAdd(p.tickets + tile, 1u) == unsigned(p.NC - 1)) ? 1u : 0u;
  cluster.sync();
  const unsigned last = *cluster.map_shared_rank(&s_last, 0);
  cluster.sync();     // rank 0 may leave only after everyone has read the flag
  if (!last) return;
  __threadfence();

  // ---- level 2: the last cluster merges the NC cluster partials, column-sliced over its blocks ----
  if (threadIdx.x < 16) {
    const int row = threadIdx.x;
    const float* ml = p.part_ml + tile * p.NC * 32;
    float M = -INFINITY;
    for (int c = 0; c < p.NC; ++c) M = fmaxf(M, __ldcg(ml + c * 32 + row * 2));
    float L = 0.f;
    for (int c = 0; c < p.NC; ++c) {
      const float mc = __ldcg(ml + c * 32 + row * 2);
      const float f = (mc == -INFINITY) ? 0.f : exp2f(mc - M);
      s_w[c][row] = f;
      L += __ldcg(ml + c * 32 + row * 2 + 1) * f;
    }
    s_l[0][row] = L;
  }
  __syncthreads();
  if (mine) {
    const float* po = p.part_o + tile * p.NC * 16 * HD;
    float acc = 0.f;
    for (int c = 0; c < p.NC; ++c) acc += __ldcg(po + (size_t(c) * 16 + mrow) * HD + c0 + mcol) * s_w[c][mrow];
    const int h = gt * 16 + mrow;
    const float L = s_l[0][mrow];
    if (h < p.G)
      p.out[(size_t(b) * p.Hq + size_t(kvh) * p.G + h) * HD + c0 + mcol] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
  }
  if (crank == 0 && threadIdx.x == 0) p.tickets[tile] = 0u;
}

template <class Kern>
static int fc_launch(Kern kern, int cl, dim3 grid, size_t smem, cudaStream_t st, bool pdl, const FcParams& p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kFcThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  int n = 1;
  if (pdl) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    n = 2;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  if (pdl) prefer_max_shared(kern);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return static_cast<int>(e);
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("flash_decode_cluster.cu")


static size_t fc_smem(int HD) { return size_t(kFcWarps) * 2 * 2 * kFcPage * HD * 2 + (16 * HD + 32) * 4; }

template <class Kern>
static int fc_prepare(Kern kern, int HD, int cl) {
  RB_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(fc_smem(HD))));
  if (cl > 8) RB_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  return 0;
}

template <class Kern>
static int fc_occupancy(Kern kern, int HD, int cl) {
  if (fc_prepare(kern, HD, cl) != 0) { (void)cudaGetLastError(); return 0; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cl * 64);
  cfg.blockDim = dim3(kFcThreads);
  cfg.dynamicSmemBytes = fc_smem(HD);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
  return n;
}

// How many clusters of `cl` blocks can be resident at once (a cluster needs `cl` free SMs of one GPC).
static int fc_max_clusters(int HD, int cl) {
  static int cached[2][2][64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int& c = cached[HD == 128 ? 1 : 0][cl == 16 ? 1 : 0][dev];
  if (c == 0) {
    int n;
    if (HD == 128) n = cl == 16 ? fc_occupancy(flash_decode_cluster_kernel<128, 16>, HD, cl)
                                : fc_occupancy(flash_decode_cluster_kernel<128, 8>, HD, cl);
    else n = cl == 16 ? fc_occupancy(flash_decode_cluster_kernel<64, 16>, HD, cl)
                      : fc_occupancy(flash_decode_cluster_kernel<64, 8>, HD, cl);
    c = n > 0 ? n : -1;
  }
  return c > 0 ? c : 0;
}

// Plan for `tiles` (= batch x kv heads x head tiles) tiles and a context of at most `max_len`
// tokens, as (cluster size << 8) | clusters per tile. Preferred: ONE cluster of 16 blocks per tile
// (a single merge level, through distributed shared memory) while a warp then owns at most four
// pages; longer contexts take several clusters of 8 per tile, one resident wave at most. 0 = the
// shape is better served by rmlx_flash_decode_paged (many tiles, or a short context).
extern "C" int rmlx_flash_decode_cluster_plan(int tiles, int max_len, int HD) {
  if (tiles < 1 || (HD != 64 && HD != 128)) return 0;
  const int pages = (max_len + kFcPage - 1) / kFcPage;
  if (pages >= 16 && pages <= 16 * kFcWarps * 4 && fc_max_clusters(HD, 16) >= tiles) return (16 << 8) | 1;
  int nc = fc_max_clusters(HD, 8) / tiles;
  const int cap = pages / 8;                     // at least one page per split
  if (nc > cap) nc = cap;
  if (nc > kFcMaxClusters) nc = kFcMaxClusters;
  return nc < 1 ? 0 : ((8 << 8) | nc);
}
extern "C" long long rmlx_flash_decode_cluster_part_o_elems(int tiles, int nc, int HD) { return 1LL * tiles * nc * 16 * HD; }
extern "C" long long rmlx_flash_decode_cluster_part_ml_elems(int tiles, int nc) { return 1LL * tiles * nc * 32; }

// `plan` from rmlx_flash_decode_cluster_plan. Scratch (clusters per tile > 1): part_o / part_ml of
// the sizes above and one zeroed ticket word per tile (left zero). head_dim 64 or 128, page 16.
extern "C" int rmlx_flash_decode_cluster(const void* q, const void* k_cache, const void* v_cache,
                                         const int* block_table, const int* seq_lens, void* out,
                                         float* part_o, float* part_ml, unsigned int* tickets, int B,
                                         int Hq, int Hkv, int HD, int max_blocks, int plan, int window,
                                         float scale, int pdl, cudaStream_t st) {
  const int nc = plan & 0xff, cl = plan >> 8;
  if (B < 1 || Hq % Hkv || nc < 1 || nc > kFcMaxClusters || (cl != 8 && cl != 16)) return -2;
  if (nc > 1 && (!part_o || !part_ml || !tickets)) return -2;
  FcParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_cache = static_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  p.block_table = block_table; p.seq_lens = seq_lens;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o; p.part_ml = part_ml; p.tickets = tickets;
  p.max_blocks = max_blocks; p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv;
  p.gtiles = (p.G + 15) / 16; p.NC = nc; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(nc * cl, Hkv * p.gtiles, B);
#define RB_FC(HD_, CL_)                                                      \
  {                                                                          \
    auto kern = flash_decode_cluster_kernel<HD_, CL_>;                       \
    const int rc = fc_prepare(kern, HD_, CL_);                               \
    if (rc != 0) return rc;                                                  \
    return fc_launch(kern, CL_, grid, fc_smem(HD_), st, pdl != 0, p);        \
  }
  if (HD == 128 && cl == 16) RB_FC(128, 16)
  if (HD == 128 && cl == 8) RB_FC(128, 8)
  if (HD == 64 && cl == 16) RB_FC(64, 16)
  if (HD == 64 && cl == 8) RB_FC(64, 8)
#undef RB_FC
  return -2;
}
