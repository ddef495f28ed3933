// Tensor-parallel GEMMs for prompt processing: the collective runs INSIDE the tcgen05 GEMM kernel
// (xgemm_kernel.cuh) over peer-mapped memory, tile by tile, instead of as a library call after it.
//
//   rmlx_tp_gemm_allreduce   row-parallel layer (attention output / FFN down projection): each rank
//                            multiplies its K-shard; accumulator tiles go from tensor memory
//                            straight into the owner rank's staging slab over NVLink, the owner
//                            sums them (+ residual) and stores the finished tile into every rank's
//                            output.  y = sum_r x_r W_r^T (+ residual), complete on every rank.
//   rmlx_tp_allgather_gemm   column-parallel layer fed by row-sharded activations (sequence
//                            parallel): ranks push their rows to everyone while the first tiles —
//                            the local rows — are already being multiplied.
//
// Every pointer array argument is a host array of ``world`` addresses that are valid in this
// process (CUDA-IPC mappings of the same buffer on each rank). Counters only grow: a call waits for
// (calls so far + 1) x the per-call count, kept per call site in ``epoch``; nothing is reset, so a
// fast rank can never race a slow one's clean-up. Waits are bounded and report through ``status``.
// Loads never touch a peer's memory and no load carries a cluster-broadcast qualifier.
//
// Replaces the reference's host-driven sequence GEMM -> commit -> wait -> RDMA all-reduce
// (crates/rmlx-nn/src/parallel.rs:619-693, crates/rmlx-distributed/src/group.rs:648-675).
#include "../kernels/xgemm_kernel.cuh"

using namespace rb;

namespace {

template <int COMM>
int launch_comm(int w_kind, int bn, bool residual, const CUtensorMap& ta, const CUtensorMap& ta2,
                const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tb, void* C,
                const void* res, int M, int N, int K, int ldc, int* status, cudaStream_t st,
                const XComm& cm) {
#define RB_C(BN_, Q_)                                                                               \
  return residual ? launch_x<BN_, Q_, false, true, COMM>(ta, ta2, tw, ts, tb, C, res, nullptr, 0, M, N, K, ldc, status, 0, st, cm) \
                  : launch_x<BN_, Q_, false, false, COMM>(ta, ta2, tw, ts, tb, C, res, nullptr, 0, M, N, K, ldc, status, 0, st, cm)
  if (bn == 256) { if (w_kind == 1) { RB_C(256, true); } else { RB_C(256, false); } }
  if (w_kind == 1) { RB_C(128, true); } else { RB_C(128, false); }
#undef RB_C
}

}  // namespace

// Staging bytes one rank needs for an [M, N] output at tile width bn (what ``stage[r]`` must hold).
extern "C" unsigned long long rmlx_tp_gemm_stage_bytes(int world, int M, int N, int bn) {
  const long long tiles = (long long)((M + kXBM - 1) / kXBM) * ((N + bn - 1) / bn);
  const long long owned = (tiles + world - 1) / world;
  return (unsigned long long)(world * owned * kXBM * bn * 2);
}

extern "C" int rmlx_tp_gemm_allreduce(int w_kind, const void* A, const void* W, const void* scales,
                                      const void* biases, const void* residual, void* const* stage,
                                      void* const* tile_flags, void* const* out, void* const* done,
                                      void* epoch, int rank, int world, int M, int N, int K, int lda,
                                      int ldc, int bn, int scatter, int* status, void* trace,
                                      cudaStream_t st) {
  // scatter != 0: GEMM + reduce-scatter. The owner of a tile (tile index modulo world; with a
  // whole number of 128-row blocks per rank that is row block b -> rank b % world, for every
  // column) keeps the reduced tile in its own output and nothing is broadcast; the ranks still
  // leave together, so the staging slabs are free for the next call.
  if (world < 1 || world > kXMaxRanks || rank < 0 || rank >= world) return -2;
  if (M < 1 || N < 8 || N % 8 || ldc % 8 || K < 8 || K % 8 || lda % 8) return -2;
  if (w_kind == 1 && K % 512) return -2;
  if (bn == 0) bn = 128;
  if (bn != 128 && bn != 256) return -2;
  CUtensorMap ta, tw, ts, tb;
  int rc = make_tmap_2d_bf16(&ta, A, uint64_t(K), uint64_t(M), uint64_t(lda) * 2, kXBK, kXBM);
  if (rc) return rc;
  rc = x_weight_maps(w_kind, W, scales, biases, uint64_t(N), K, bn, &tw, &ts, &tb);
  if (rc) return rc;
  XComm cm;
  cm.rank = rank; cm.world = world;
  cm.epoch = static_cast<uint32_t*>(epoch);
  cm.trace = static_cast<unsigned long long*>(trace);   // optional [grid][8] phase timestamps
  const int tiles = ((M + kXBM - 1) / kXBM) * ((N + bn - 1) / bn);
  cm.tiles_owned_max = (tiles + world - 1) / world;
  cm.scatter = scatter != 0;
  for (int p = 0; p < world; ++p) {
    cm.stage[p] = static_cast<__nv_bfloat16*>(stage[p]);
    cm.tile_flags[p] = static_cast<uint32_t*>(tile_flags[p]);
    cm.out[p] = static_cast<__nv_bfloat16*>(out[p]);
    cm.done[p] = static_cast<uint32_t*>(done[p]);
  }
  return launch_comm<kCommReduce>(w_kind, bn, residual != nullptr, ta, ta, tw, ts, tb, out[rank],
                                  residual, M, N, K, ldc, status, st, cm);
}

// a_full[r]: rank r's gathered buffer, 2 x [world*shard_rows, K] bf16 (two parities);
// ready[r]: rank r's counters, one per 128-row block of the gathered matrix.
extern "C" int rmlx_tp_allgather_gemm(int w_kind, const void* a_shard, int lda_shard, int shard_rows,
                                      void* const* a_full, void* const* ready, void* epoch,
                                      const void* W, const void* scales, const void* biases, void* C,
                                      const void* residual, int rank, int world, int N, int K,
                                      int ldc, int bn, int* status, void* trace, cudaStream_t st) {
  if (world < 1 || world > kXMaxRanks || rank < 0 || rank >= world) return -2;
  if (shard_rows < kXBM || shard_rows % kXBM || lda_shard % 8 || K < 8 || K % 8 || N < 1) return -2;
  if (w_kind == 1 && K % 512) return -2;
  if (bn == 0) bn = 128;
  if (bn != 128 && bn != 256) return -2;
  const int M = world * shard_rows;
  CUtensorMap ta, ta2, tw, ts, tb;
  const __nv_bfloat16* full = static_cast<const __nv_bfloat16*>(a_full[rank]);
  int rc = make_tmap_2d_bf16(&ta, full, uint64_t(K), uint64_t(M), uint64_t(K) * 2, kXBK, kXBM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&ta2, full + size_t(M) * K, uint64_t(K), uint64_t(M), uint64_t(K) * 2, kXBK, kXBM);
  if (rc) return rc;
  rc = x_weight_maps(w_kind, W, scales, biases, uint64_t(N), K, bn, &tw, &ts, &tb);
  if (rc) return rc;
  XComm cm;
  cm.rank = rank; cm.world = world;
  cm.epoch = static_cast<uint32_t*>(epoch);
  cm.trace = static_cast<unsigned long long*>(trace);   // optional [grid][8] phase timestamps
  cm.a_shard = static_cast<const __nv_bfloat16*>(a_shard);
  cm.lda_shard = lda_shard; cm.shard_rows = shard_rows;
  for (int p = 0; p < world; ++p) {
    cm.a_full[p] = static_cast<__nv_bfloat16*>(a_full[p]);
    cm.ready[p] = static_cast<uint32_t*>(ready[p]);
  }
  return launch_comm<kCommGather>(w_kind, bn, residual != nullptr, ta, ta2, tw, ts, tb, C, residual, M,
                                  N, K, ldc, status, st, cm);
}
