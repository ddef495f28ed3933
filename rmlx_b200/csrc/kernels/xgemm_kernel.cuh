// The generalised tcgen05 GEMM kernel (see xgemm_tcgen05.cu for the plain entry points and
// ../comm/tp_gemm.cu for the tensor-parallel ones). C = A · W^T with
//   * W bf16 (TMA-fed) or MLX-affine Q4 dequantised inside the main loop by eight dequant warps;
//   * GROUPED: rows of A sorted by expert, tile table derived on the device from offsets[E+1];
//   * swiglu: a tile holds BN/2 gate rows and the matching BN/2 up rows of W; the epilogue writes
//     silu(gate) * up straight from the fp32 accumulators;
//   * COMM = kCommReduce: this rank holds a K-shard; every finished accumulator tile is stored
//     straight into the staging slab of the rank that owns the tile (peer stores over NVLink; a
//     signalling warp publishes a release counter per tile); four collective warps of the owner
//     sum the world's partials (+ residual) and store the finished tile into every rank's output —
//     reduce-scatter and all-gather of an all-reduce, both inside the GEMM kernel, running
//     alongside the tiles still being multiplied;
//   * COMM = kCommGather: A is row-sharded over the ranks; the collective warps push this rank's
//     rows into every peer's gathered copy in 8-row chunks with a counter per 128-row block; the
//     TMA producer starts with the local rows (row-block-major tile order, rotated by rank) and
//     waits for a block's counter before its first load of remote rows.
// Every wait — mbarrier or peer counter — is bounded; a timeout sets the status word and the CTA
// drains and frees its tensor memory. Peer data is only ever *pushed* (plain stores); loads are
// always from this GPU's memory.
#pragma once
#include <cuda.h>
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include "../common/tensormap.cuh"

namespace rb {

constexpr int kXBM = 128;
constexpr int kXBK = 64;
constexpr int kXMaxExperts = 256;
constexpr int kXMaxRanks = 8;
constexpr int kCommNone = 0, kCommReduce = 1, kCommGather = 2;
constexpr int kGatherChunkRows = 8;
constexpr int kDqWarps = 8;          // dequant warps of the Q4 main loop (two per SM sub-partition)
constexpr int kCommThreads = 160;   // collective modes: four reducer/pusher warps + one signalling warp

struct XComm {
  int rank = 0, world = 1;
  uint32_t* epoch = nullptr;                 // local: [0] calls completed, [1] exit ticket
  // reduce
  __nv_bfloat16* stage[kXMaxRanks] = {};     // rank p's staging slab [world][tiles_owned_max][128*BN]
  uint32_t* tile_flags[kXMaxRanks] = {};     // rank p's arrival counter per owned tile
  __nv_bfloat16* out[kXMaxRanks] = {};       // rank p's output matrix [M, ldc]
  uint32_t* done[kXMaxRanks] = {};           // rank p's count of finished tiles
  int tiles_owned_max = 0;
  int scatter = 0;                           // 1: reduce-scatter (the owner keeps the finished tile, no broadcast)
  // gather
  const __nv_bfloat16* a_shard = nullptr;    // this rank's rows [shard_rows, lda_shard]
  int lda_shard = 0, shard_rows = 0;
  __nv_bfloat16* a_full[kXMaxRanks] = {};    // rank p's gathered copy, two parities [2][M][K]
  uint32_t* ready[kXMaxRanks] = {};          // rank p's counter per 128-row block
  unsigned long long* trace = nullptr;       // optional [grid][8] timestamps (see x_trace)
};

// MT = 2: a tile is two stacked 128-row blocks of A against ONE staged block of W, i.e. two
// accumulators per dequantised operand stage — the dequant warps' work per multiply-add halves.
template <int BN, bool WQ4, int MT = 1>
struct XSmem {
  static constexpr int kStages = MT == 2 ? 3 : (WQ4 ? ((BN >= 256) ? 3 : 5) : ((BN >= 256) ? 4 : 6));
  static constexpr int kRawStages = 4;
  static constexpr int kStageA = MT * kXBM * kXBK * 2;
  static constexpr int kStageB = BN * kXBK * 2;
  static constexpr int kStageRaw = BN * 32;          // 64 nibbles per row
  static constexpr int kScaleSlot = 2 * BN * 16;     // scales + biases for 8 k-blocks
  static constexpr int kBytes = kStages * (kStageA + kStageB) +
                                (WQ4 ? kRawStages * kStageRaw + 2 * kScaleSlot : 0) + 1024 + 512 +
                                (kXMaxExperts + 2) * 8;
  static constexpr int kThreads = WQ4 ? 192 + 32 * kDqWarps : 192;
};

struct XTile {
  int a_row0;     // first row of the A/C tile
  int row_end;    // rows >= row_end are not stored
  int w_row0;     // first row of the W tile (in the stacked weight)
  int c_col0;     // first output column
};

// tile id -> coordinates. Plain: column-block major so consecutive CTAs share a W tile; ``rot``
// rotates the row blocks so that a rank starts with the rows it already holds (gather mode).
template <int BN, bool GROUPED, bool ROW_MAJOR = false, int MT = 1>
__device__ __forceinline__ XTile x_tile(int tile, int M, int N, int tiles_m, int tiles_n,
                                        const int* s_off, const int* s_tprefix, int E, int rot = 0,
                                        int half = 0) {
  // half = 1 (SwiGLU mode): a tile holds BN/2 gate rows and the matching BN/2 up rows of W and
  // produces BN/2 output columns; w_row0 is the gate row, the up row sits N/2 further.
  XTile t;
  if (!GROUPED) {
    // ROW_MAJOR (gather mode): all column tiles of a row block before the next row block, so the
    // rotation really puts every tile of the local rows first
    int tm = (ROW_MAJOR ? tile / tiles_n : tile % tiles_m) + rot;
    if (tm >= tiles_m) tm -= tiles_m;
    const int tn = ROW_MAJOR ? tile % tiles_n : tile / tiles_m;
    t.a_row0 = tm * (kXBM * MT); t.row_end = M; t.w_row0 = tn * (BN >> half); t.c_col0 = tn * (BN >> half);
  } else {
    int e = 0;
    while (e + 1 < E && s_tprefix[e + 1] <= tile) ++e;
    while (s_tprefix[e + 1] <= tile) ++e;                 // skips empty experts
    const int local = tile - s_tprefix[e];
    const int rows = s_off[e + 1] - s_off[e];
    const int mt_e = (rows + kXBM * MT - 1) / (kXBM * MT);
    const int nt = local / mt_e, mt = local % mt_e;
    t.a_row0 = s_off[e] + mt * (kXBM * MT); t.row_end = s_off[e + 1];
    t.w_row0 = e * N + nt * (BN >> half); t.c_col0 = nt * (BN >> half);
  }
  return t;
}

// Optional phase trace of the collective modes: slot k of this CTA's row gets the global timer
// (0 start, 1 last MMA issued, 2 epilogue done, 3 collective warps done, 4 exit).
template <int COMM>
__device__ __forceinline__ void x_trace(const XComm& cm, int k) {
  if (COMM != kCommNone && cm.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    cm.trace[blockIdx.x * 8 + k] = t;
  }
}

// Barrier over the four epilogue warps, built on an mbarrier so that it is bounded like every other
// wait: if a warp left early after a timeout, the rest give up too instead of waiting for it.
__device__ __forceinline__ bool epi_sync(uint64_t* bar, uint32_t& phase, volatile uint32_t* abort_flag,
                                         uint32_t limit) {
  mbar_arrive(bar);
  const bool ok = mbar_wait(bar, phase, abort_flag, limit);
  phase ^= 1u;
  return ok;
}

// Owner-side sum of one tile: a warp covers 4 rows x 8 sixteen-byte groups per step (64-byte runs
// of the staging layout in, 128-byte runs of output rows out) and keeps U steps x W sources of loads
// in flight. The residual is added once, here.
template <int BN, bool RESIDUAL, int W, int U>
__device__ __forceinline__ void x_reduce_tile(const XComm& cm, const __nv_bfloat16* sl, size_t src_stride,
                                              const XTile& t, int M, int N, int ldc,
                                              const __nv_bfloat16* residual, int cw, int lane) {
  constexpr int GB = BN / 64;
  constexpr int STEPS = (kXBM / 4) * GB;
  for (int step0 = cw * U; step0 < STEPS; step0 += 4 * U) {
    uint4 pv[U][W];
    uint4 rv[U];
    size_t off[U];
    bool inb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int step = step0 + u;
      const int g = (step % GB) * 8 + (lane & 7), r = (step / GB) * 4 + (lane >> 3);
#pragma unroll
      for (int s = 0; s < W; ++s)
        if (s < cm.world)
          pv[u][s] = __ldcg(reinterpret_cast<const uint4*>(sl + s * src_stride + (size_t(g) * kXBM + r) * 8));
      const int row = t.a_row0 + r, col = t.c_col0 + g * 8;
      inb[u] = row < M && col < N;              // N is a multiple of 8 (checked by the launcher)
      off[u] = size_t(row) * ldc + col;
      rv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (RESIDUAL && inb[u]) rv[u] = *reinterpret_cast<const uint4*>(residual + off[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float f[8] = {bf16lo(rv[u].x), bf16hi(rv[u].x), bf16lo(rv[u].y), bf16hi(rv[u].y),
                    bf16lo(rv[u].z), bf16hi(rv[u].z), bf16lo(rv[u].w), bf16hi(rv[u].w)};
#pragma unroll
      for (int s = 0; s < W; ++s) {
        if (s < cm.world) {
          const uint4 v = pv[u][s];
          f[0] += bf16lo(v.x); f[1] += bf16hi(v.x); f[2] += bf16lo(v.y); f[3] += bf16hi(v.y);
          f[4] += bf16lo(v.z); f[5] += bf16hi(v.z); f[6] += bf16lo(v.w); f[7] += bf16hi(v.w);
        }
      }
      if (inb[u]) {
        uint4 o;
        o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
        o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
        if (cm.scatter) {
          *reinterpret_cast<uint4*>(cm.out[cm.rank] + off[u]) = o;
        } else {
          for (int pi = 0; pi < cm.world; ++pi) {
            int p = cm.rank + pi; if (p >= cm.world) p -= cm.world;
            *reinterpret_cast<uint4*>(cm.out[p] + off[u]) = o;
          }
        }
      }
    }
  }
}

template <int BN, bool WQ4, bool GROUPED, bool RESIDUAL, int COMM, int MT>
__global__ void __launch_bounds__((XSmem<BN, WQ4>::kThreads + (COMM != kCommNone ? kCommThreads : 0)), 1)
xgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a2,
             const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
             const __grid_constant__ CUtensorMap tmap_b, __nv_bfloat16* __restrict__ C,
             const __nv_bfloat16* __restrict__ residual, const int* __restrict__ offsets, int E, int M,
             int N, int K, int ldc, int* __restrict__ status, const XComm cm, int swiglu) {
  static_assert(COMM == kCommNone || !GROUPED, "collective modes are for plain GEMMs");
  static_assert(MT == 1 || (COMM == kCommNone && 2 * BN * MT <= 512), "stacked tiles: no collective modes");
  using S = XSmem<BN, WQ4, MT>;
  constexpr int STAGES = S::kStages, RAW = S::kRawStages;
  // a role may be waiting, through the pipeline, on a peer that started late: be more patient then
  constexpr uint32_t LIM = (COMM == kCommNone) ? kMbarPollLimit : (kMbarPollLimit << 4);
  constexpr int kCommWarp0 = S::kThreads / 32;          // first of the five collective-mode warps
  constexpr uint32_t TMEM_COLS = (2 * BN * MT <= 32) ? 32 : 2 * BN * MT;
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
  uint64_t* sig_full = acc_empty + 2;           // [2] partial tile stored by the epilogue warps
  uint64_t* sig_free = sig_full + 2;            // [2] its signal has gone out
  uint64_t* comm_mb = sig_free + 2;             // [1] collective-warp barrier
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(comm_mb + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* peer_fail = tmem_slot + 2;
  int* s_off = reinterpret_cast<int*>(after + 512);          // [E+1]
  int* s_tprefix = s_off + kXMaxExperts + 1;                 // [E+1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN;
  int tiles_m = (M + kXBM * MT - 1) / (kXBM * MT);
  const int num_kb = (K + kXBK - 1) / kXBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, 1); mbar_init(bq_full + i, kDqWarps); }
    for (int i = 0; i < RAW; ++i) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, kDqWarps); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(sc_full + i, 1); mbar_init(sc_empty + i, kDqWarps);
      mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 4);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(sig_full + i, 128); mbar_init(sig_free + i, 1); }
    mbar_init(comm_mb, 128);
    *abort_flag = 0u;
    *peer_fail = 0u;
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
        acc += ((s_off[e + 1] - s_off[e] + kXBM * MT - 1) / (kXBM * MT)) * tiles_n;
      }
      s_tprefix[E] = acc;
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? s_tprefix[E] : tiles_m * tiles_n;
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) x_trace<COMM>(cm, 0);
  // collective modes: calls completed so far on this site; counters only grow, so a call waits
  // for (epoch+1) x the per-call increment and nothing is ever reset.
  const uint32_t e1 = (COMM != kCommNone) ? cm.epoch[0] + 1u : 0u;
  const int rot = (COMM == kCommGather) ? (cm.rank * cm.shard_rows) / kXBM : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      const CUtensorMap* ta = (COMM == kCommGather && (e1 & 1u) == 0u) ? &tmap_a2 : &tmap_a;
      tma_prefetch_desc(ta);
      tma_prefetch_desc(&tmap_w);
      if (!GROUPED) pdl_wait();
      int stage = 0, rstage = 0, sslot = 0;
      uint32_t phase = 0, rphase = 0, sphase = 0;
      bool ok = true;
      int ready_mb = -1;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const XTile t = x_tile<BN, GROUPED, COMM == kCommGather, MT>(tile, M, N, tiles_m, tiles_n, s_off, s_tprefix, E, rot, swiglu);
        if (COMM == kCommGather) {
          const int mb = t.a_row0 / kXBM;
          if (mb != ready_mb) {
            // rows of this block are pushed by their owner (this rank included) in 8-row chunks
            if (!wait_flag_ge(cm.ready[cm.rank] + mb, e1 * (kXBM / kGatherChunkRows))) {
              *peer_fail = 1u; *abort_flag = 1u; ok = false; break;
            }
            asm volatile("fence.proxy.async;" ::: "memory");   // peer stores -> TMA reads
            ready_mb = mb;
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (WQ4) {
            if ((kb & 7) == 0) {
              if (!mbar_wait(sc_empty + sslot, sphase ^ 1u, abort_flag, LIM)) { ok = false; break; }
              mbar_arrive_expect_tx(sc_full + sslot, S::kScaleSlot);
              char* sd = sScale + sslot * S::kScaleSlot;
              tma_load_2d(sd, &tmap_s, sc_full + sslot, kb, t.w_row0);
              tma_load_2d(sd + BN * 16, &tmap_b, sc_full + sslot, kb, t.w_row0);
              if (swiglu) {     // the maps' boxes are BN/2 rows tall in this mode: second half = up rows
                tma_load_2d(sd + BN * 8, &tmap_s, sc_full + sslot, kb, t.w_row0 + N / 2);
                tma_load_2d(sd + BN * 16 + BN * 8, &tmap_b, sc_full + sslot, kb, t.w_row0 + N / 2);
              }
              if (++sslot == 2) { sslot = 0; sphase ^= 1u; }
            }
            if (!mbar_wait(raw_empty + rstage, rphase ^ 1u, abort_flag, LIM)) { ok = false; break; }
            mbar_arrive_expect_tx(raw_full + rstage, S::kStageRaw);
            tma_load_2d(sRaw + rstage * S::kStageRaw, &tmap_w, raw_full + rstage, kb * 32, t.w_row0);
            if (swiglu)
              tma_load_2d(sRaw + rstage * S::kStageRaw + BN * 16, &tmap_w, raw_full + rstage, kb * 32, t.w_row0 + N / 2);
            if (++rstage == RAW) { rstage = 0; rphase ^= 1u; }
          }
          if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag, LIM)) { ok = false; break; }
          mbar_arrive_expect_tx(full + stage, S::kStageA + (WQ4 ? 0 : S::kStageB));
#pragma unroll
          for (int mh = 0; mh < MT; ++mh)
            tma_load_2d(sA + stage * S::kStageA + mh * (kXBM * kXBK * 2), ta, full + stage, kb * kXBK,
                        t.a_row0 + mh * kXBM);
          if (!WQ4) {
            tma_load_2d(sB + stage * S::kStageB, &tmap_w, full + stage, kb * kXBK, t.w_row0);
            if (swiglu)
              tma_load_2d(sB + stage * S::kStageB + BN * 64, &tmap_w, full + stage, kb * kXBK, t.w_row0 + N / 2);
          }
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
        if (!mbar_wait(acc_empty + acc, acc_phase ^ 1u, abort_flag, LIM)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * (BN * MT);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase, abort_flag, LIM)) { ok = false; break; }
          if (WQ4 && !mbar_wait(bq_full + stage, phase, abort_flag, LIM)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kStageA);
          const uint32_t b_addr = smem_u32(sB + stage * S::kStageB);
#pragma unroll
          for (int k = 0; k < kXBK / 16; ++k)
#pragma unroll
            for (int mh = 0; mh < MT; ++mh)
              tc_mma_f16(d_tmem + mh * BN, umma_desc_sw128_kmajor(a_addr + mh * (kXBM * kXBK * 2) + k * 32),
                         umma_desc_sw128_kmajor(b_addr + k * 32), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(empty + stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(acc_full + acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      x_trace<COMM>(cm, 1);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int et = threadIdx.x - 64;            // 0..127 over the epilogue warps
    (void)et;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    if (RESIDUAL && !GROUPED) pdl_wait();

    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const XTile t = x_tile<BN, GROUPED, COMM == kCommGather, MT>(tile, M, N, tiles_m, tiles_n, s_off, s_tprefix, E, rot, swiglu);
      if (!mbar_wait(acc_full + acc, acc_phase, abort_flag, LIM)) { ok = false; break; }
      tc_fence_after_sync();
      int row = t.a_row0 + q * 32 + lane;
      uint32_t t_row = tmem_base + acc * (BN * MT) + (uint32_t(q * 32) << 16);
      if (COMM == kCommReduce) {
        // partial tile -> the owner's staging slab, laid out so that each warp-wide store is one
        // contiguous 512-byte run: 16-byte group (c*4+v) of row r sits at ((c*4+v)*128 + r)*16.
        const int owner = tile % cm.world, slot = tile / cm.world;
        __nv_bfloat16* sbase = cm.stage[owner] +
                               (size_t(cm.rank) * cm.tiles_owned_max + slot) * size_t(kXBM * BN);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
            *reinterpret_cast<uint4*>(sbase + (size_t(c * 4 + v) * kXBM + q * 32 + lane) * 8) = o;
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + acc);
        // hand the tile to the signalling warp: it makes the stores visible system-wide and bumps
        // the owner's counter, off this warp's critical path (the slot is free again once the
        // signal two tiles back has gone out)
        if (!mbar_wait(sig_free + acc, acc_phase ^ 1u, abort_flag, LIM)) { ok = false; break; }
        mbar_arrive(sig_full + acc);
      } else {
#pragma unroll 1
       for (int mh = 0; mh < MT; ++mh, row += kXBM, t_row += BN) {      // stacked 128-row blocks
        if (swiglu) {
        // accumulator columns [0, BN/2) are the gate, [BN/2, BN) the up projection of the same
        // output columns: out = silu(gate) * up, straight from tensor memory
        const int n_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_row + c * 32, rg);
          tmem_ld_32x32(t_row + BN / 2 + c * 32, ru);
          tmem_ld_wait();
          const int col0 = t.c_col0 + c * 32;
          if (row < t.row_end && col0 < n_out) {
            __nv_bfloat16* dst = C + size_t(row) * ldc + col0;
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float g = __uint_as_float(rg[j]);
              f[j] = g / (1.f + __expf(-g)) * __uint_as_float(ru[j]);
            }
            if (col0 + 32 <= n_out) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack_bf16(f[v * 8 + 0], f[v * 8 + 1]); o.y = pack_bf16(f[v * 8 + 2], f[v * 8 + 3]);
                o.z = pack_bf16(f[v * 8 + 4], f[v * 8 + 5]); o.w = pack_bf16(f[v * 8 + 6], f[v * 8 + 7]);
                *reinterpret_cast<uint4*>(dst + v * 8) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < n_out) dst[j] = __float2bfloat16_rn(f[j]);
            }
          }
        }
        } else {
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
        }
       }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + acc);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (et == 0) x_trace<COMM>(cm, 2);
  } else if (COMM == kCommReduce && warp == kCommWarp0 + 4) {
    // ------------------------------------------------------------------ signalling warp
    if (lane == 0) {
      int acc = 0;
      uint32_t ph = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (!mbar_wait(sig_full + acc, ph, abort_flag, LIM)) break;
        __threadfence_system();
        red_release_sys_add(cm.tile_flags[tile % cm.world] + tile / cm.world, 1u);
        mbar_arrive(sig_free + acc);
        if (++acc == 2) { acc = 0; ph ^= 1u; }
      }
    }
  } else if (COMM != kCommNone && warp >= kCommWarp0 && warp < kCommWarp0 + 4) {
    // ------------------------------------------------------------------ collective warps (4)
    const int ct = threadIdx.x - kCommWarp0 * 32;     // 0..127
    uint32_t cphase = 0;
    if (COMM == kCommGather) {
      // push this rank's rows to every rank's gathered copy (its own included), 8 rows at a time,
      // four 16-byte loads in flight per thread
      const int chunks = cm.shard_rows / kGatherChunkRows;
      const int vec_per_row = K / 8;
      const int vecs = kGatherChunkRows * vec_per_row;
      const size_t parity_off = ((e1 & 1u) == 0u) ? size_t(M) * K : 0;
      for (int ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
        const int r0 = ch * kGatherChunkRows;
        const int grow0 = cm.rank * cm.shard_rows + r0;
        for (int i0 = ct; i0 < vecs; i0 += 4 * 128) {
          uint4 v[4];
          size_t doff[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 128;
            if (i < vecs) {
              const int r = i / vec_per_row, c = i % vec_per_row;
              v[u] = __ldcs(reinterpret_cast<const uint4*>(cm.a_shard + size_t(r0 + r) * cm.lda_shard + c * 8));
              doff[u] = parity_off + size_t(grow0 + r) * K + c * 8;
            }
          }
          for (int pi = 0; pi < cm.world; ++pi) {
            int p = cm.rank + pi; if (p >= cm.world) p -= cm.world;
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (i0 + u * 128 < vecs) *reinterpret_cast<uint4*>(cm.a_full[p] + doff[u]) = v[u];
          }
        }
        if (!epi_sync(comm_mb, cphase, abort_flag, LIM)) break;
        if (ct == 0) {
          __threadfence_system();
          for (int p = 0; p < cm.world; ++p) red_release_sys_add(cm.ready[p] + grow0 / kXBM, 1u);
        }
      }
      if (ct == 0) x_trace<COMM>(cm, 3);
    } else {
      // owner side, concurrent with the main loop: sum the world's partials of each tile this rank
      // owns, add the residual once, store the finished tile into every rank's output, count it as
      // done everywhere. A warp covers 4 rows x 8 groups per step: 64-byte runs of the staging
      // layout in, 128-byte runs of output rows out.
      const int cw = ct >> 5;
      const int n_owned = (num_tiles - cm.rank + cm.world - 1) / cm.world;
      const size_t src_stride = size_t(cm.tiles_owned_max) * size_t(kXBM * BN);
      int tiles_done = 0;
      for (int j = blockIdx.x; j < n_owned; j += gridDim.x) {
        if (ct == 0 && !wait_flag_ge(cm.tile_flags[cm.rank] + j, e1 * uint32_t(cm.world), kPeerPollLimit << 2)) {
          *peer_fail = 1u; *abort_flag = 1u;
        }
        if (!epi_sync(comm_mb, cphase, abort_flag, LIM) || *abort_flag) break;
        const int tile = j * cm.world + cm.rank;
        const XTile t = x_tile<BN, false>(tile, M, N, tiles_m, tiles_n, s_off, s_tprefix, E, 0);
        const __nv_bfloat16* sl = cm.stage[cm.rank] + size_t(j) * size_t(kXBM * BN);
        if (cm.world <= 2) x_reduce_tile<BN, RESIDUAL, 2, 4>(cm, sl, src_stride, t, M, N, ldc, residual, cw, lane);
        else if (cm.world <= 4) x_reduce_tile<BN, RESIDUAL, 4, 2>(cm, sl, src_stride, t, M, N, ldc, residual, cw, lane);
        else x_reduce_tile<BN, RESIDUAL, 8, 1>(cm, sl, src_stride, t, M, N, ldc, residual, cw, lane);
        ++tiles_done;
      }
      // one visibility fence and one count per peer for everything this CTA reduced
      if (epi_sync(comm_mb, cphase, abort_flag, LIM) && ct == 0 && tiles_done > 0) {
        __threadfence_system();
        for (int p = 0; p < cm.world; ++p) red_release_sys_add(cm.done[p], uint32_t(tiles_done));
      }
      if (ct == 0) x_trace<COMM>(cm, 3);
      // every tile of the result has landed here before this rank's kernel ends
      if (ct == 0 && !*abort_flag) {
        if (!wait_flag_ge(cm.done[cm.rank], e1 * uint32_t(num_tiles), kPeerPollLimit << 2)) {
          *peer_fail = 1u; *abort_flag = 1u;
        }
      }
    }
  } else if (WQ4 && warp < 6 + kDqWarps) {
    // ------------------------------------------------------------------ dequant (warps 6..13)
    const int dt = threadIdx.x - 192;   // 0 .. 32*kDqWarps-1
    int stage = 0, rstage = 0, sslot = 0;
    uint32_t phase = 0, rphase = 0, sphase = 0;
    bool ok = true;
    // Static work split: item = (row of the W tile, which 32-element half of the 64-wide k-block);
    // consecutive threads take consecutive 16-byte pieces of the packed tile (conflict-free loads),
    // and a row's 8 group scales/biases stay in registers for 8 k-blocks.
    constexpr int ITEMS = (BN * 2 + 32 * kDqWarps - 1) / (32 * kDqWarps);
    const __nv_bfloat162 k128 = __float2bfloat162_rn(128.f);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb8 = 0; kb8 < num_kb && ok; kb8 += 8) {     // K % 512 == 0: whole groups of 8
        if (!mbar_wait(sc_full + sslot, sphase, abort_flag, LIM)) { ok = false; break; }
        uint4 sv[ITEMS], bv[ITEMS];
        const char* scb = sScale + sslot * S::kScaleSlot;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          const int item = it * (32 * kDqWarps) + dt;
          if (item < BN * 2) {
            sv[it] = *reinterpret_cast<const uint4*>(scb + (item >> 1) * 16);
            bv[it] = *reinterpret_cast<const uint4*>(scb + BN * 16 + (item >> 1) * 16);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sc_empty + sslot);       // the slot can be refilled already
        if (++sslot == 2) { sslot = 0; sphase ^= 1u; }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (!mbar_wait(raw_full + rstage, rphase, abort_flag, LIM)) { ok = false; break; }
          if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag, LIM)) { ok = false; break; }  // B slot free
          const char* raw = sRaw + rstage * S::kStageRaw;
          char* bst = sB + stage * S::kStageB;
#pragma unroll
          for (int it = 0; it < ITEMS; ++it) {
            const int item = it * (32 * kDqWarps) + dt;
            if (item < BN * 2) {
              const int r = item >> 1, h = item & 1;
              const uint4 wv = *reinterpret_cast<const uint4*>(raw + item * 16);
              const uint32_t sw = (kk >> 1) == 0 ? sv[it].x : (kk >> 1) == 1 ? sv[it].y : (kk >> 1) == 2 ? sv[it].z : sv[it].w;
              const uint32_t bw = (kk >> 1) == 0 ? bv[it].x : (kk >> 1) == 1 ? bv[it].y : (kk >> 1) == 2 ? bv[it].z : bv[it].w;
              const uint32_t s2u = __byte_perm(sw, 0u, (kk & 1) ? 0x3232u : 0x1010u);
              const uint32_t b2u = __byte_perm(bw, 0u, (kk & 1) ? 0x3232u : 0x1010u);
              const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&s2u);
              const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&b2u);
              const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t w = words[j], w4 = w >> 4;
                // byte b of the word holds elements 2b (low nibble) and 2b+1 (high nibble): pick the
                // byte from w and from w>>4 into the two halves, keep the low nibbles, and drop them
                // into the mantissa of 128.0 (128 + q is exact in bf16)
                uint32_t p0 = (__byte_perm(w, w4, 0x0400u) & 0x000f000fu) | 0x43004300u;
                uint32_t p1 = (__byte_perm(w, w4, 0x0501u) & 0x000f000fu) | 0x43004300u;
                uint32_t p2 = (__byte_perm(w, w4, 0x0602u) & 0x000f000fu) | 0x43004300u;
                uint32_t p3 = (__byte_perm(w, w4, 0x0703u) & 0x000f000fu) | 0x43004300u;
                __nv_bfloat162 v0 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p0), k128), s2, b2);
                __nv_bfloat162 v1 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p1), k128), s2, b2);
                __nv_bfloat162 v2 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p2), k128), s2, b2);
                __nv_bfloat162 v3 = __hfma2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&p3), k128), s2, b2);
                uint4 o;   // natural k order: (k0,k1) (k2,k3) (k4,k5) (k6,k7)
                o.x = *reinterpret_cast<uint32_t*>(&v0); o.y = *reinterpret_cast<uint32_t*>(&v1);
                o.z = *reinterpret_cast<uint32_t*>(&v2); o.w = *reinterpret_cast<uint32_t*>(&v3);
                const int c = h * 4 + j;                 // 16-byte chunk of the 128-byte row
                *reinterpret_cast<uint4*>(bst + r * 128 + ((c ^ (r & 7)) << 4)) = o;
              }
            }
          }
          fence_proxy_async_smem();     // generic-proxy stores -> visible to the tensor core's reads
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(bq_full + stage);
            mbar_arrive(raw_empty + rstage);
          }
          if (++rstage == RAW) { rstage = 0; rphase ^= 1u; }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) { tc_fence_after_sync(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (threadIdx.x == 0) {
    x_trace<COMM>(cm, 4);
    if (*abort_flag && status) atomicExch(status, *peer_fail ? kStatusPeerTimeout : kStatusMbarTimeout);
    if (COMM != kCommNone) {
      // the last CTA to leave advances the site's epoch for the next call
      __threadfence();
      if (atomicAdd(cm.epoch + 1, 1u) == gridDim.x - 1) { cm.epoch[1] = 0u; cm.epoch[0] = e1; }
    }
  }
  pdl_launch_dependents();
}

template <int BN, bool WQ4, bool GROUPED, bool RESIDUAL, int COMM = kCommNone, int MT = 1>
static int launch_x(const CUtensorMap& ta, const CUtensorMap& ta2, const CUtensorMap& tw,
                    const CUtensorMap& ts, const CUtensorMap& tb, void* C, const void* residual,
                    const int* offsets, int E, int M, int N, int K, int ldc, int* status, int pdl,
                    cudaStream_t st, const XComm& cm = XComm(), int swiglu = 0) {
  using S = XSmem<BN, WQ4, MT>;
  auto kern = xgemm_kernel<BN, WQ4, GROUPED, RESIDUAL, COMM, MT>;
  RB_CHECK(set_max_smem(kern, S::kBytes));
  int tiles = ((M + kXBM * MT - 1) / (kXBM * MT)) * ((N + BN - 1) / BN);
  if (GROUPED) tiles += E * ((N + BN - 1) / BN);   // upper bound: every group may add a ragged tile
  const int grid = tiles < sm_count() ? (tiles > 0 ? tiles : 1) : sm_count();
  return launch(kern, dim3(grid), dim3(S::kThreads + (COMM != kCommNone ? kCommThreads : 0)), size_t(S::kBytes), st, pdl != 0, ta, ta2, tw, ts, tb,
                static_cast<__nv_bfloat16*>(C), static_cast<const __nv_bfloat16*>(residual), offsets, E,
                M, N, K, ldc, status, cm, swiglu);
}

// Tensor maps of the weight operand (and of its scales/biases for Q4).
static inline int x_weight_maps(int w_kind, const void* W, const void* scales, const void* biases,
                                uint64_t rowsW, int K, int bn, CUtensorMap* tw, CUtensorMap* ts,
                                CUtensorMap* tb) {
  int rc;
  if (w_kind == 0) {
    rc = make_tmap_2d_bf16(tw, W, uint64_t(K), rowsW, uint64_t(K) * 2, kXBK, bn);
    if (rc) return rc;
    *ts = *tw; *tb = *tw;
    return 0;
  }
  rc = make_tmap_2d(tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, uint64_t(K) / 2, rowsW, uint64_t(K) / 2,
                    32, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap_2d(ts, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, scales, uint64_t(K) / 64, rowsW,
                    uint64_t(K) / 64 * 2, 8, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  return make_tmap_2d(tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, biases, uint64_t(K) / 64, rowsW,
                      uint64_t(K) / 64 * 2, 8, bn, CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace rb
