// All-reduce done by the NVLink switch: the operands sit at the same offset of the symmetric heap
// on every rank, the heap segment is bound to a multicast object, and each rank reduces its own
// slice with `multimem.ld_reduce` (the switch fetches the slice from every rank and returns the
// sum) and writes it back with `multimem.st` (the switch stores it into every rank's copy). Two
// crossings of the fabric per element, no rank reads another rank's memory with ordinary loads.
//
// Counterpart of the reference's ring / tree all-reduce over RDMA
// (crates/rmlx-distributed/src/group.rs:348-504), which has no in-fabric reduction to use.
//
// Flags (one small area per rank, peer-mapped, plain release adds): block 0 of every rank tells every
// rank that this rank's input is complete, waits for all ranks and opens a local gate for its
// sibling blocks; the last block to finish tells every rank that this rank's slice has been
// broadcast and waits for all ranks. Counters only grow: the call number lives in the flag area,
// is read by every block at its start and advanced by the last block to leave, so captured and
// eager calls, and calls with different grids, can be mixed. Every wait is bounded and reports
// through a status word.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"

namespace rb {

constexpr int kNvlsMaxWorld = 8;
constexpr int kNvlsMaxBlocks = 64;
// flag area (u32 words): 0 input-ready counter, 1 done counter (both written by every rank),
// 2 call number, 3 exit ticket, 4 local gate (this rank only)
constexpr int kNvlsFlagWords = 8;

__device__ int g_nvls_status = 0;

struct NvlsPeers {
  uint32_t* flags[kNvlsMaxWorld];   // every rank's flag area, peer-mapped; index = rank
  int rank, world;
};

__device__ __forceinline__ uint4 mm_ld_reduce_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// mc: multicast address of the operand (16-byte aligned); nvec: 16-byte vectors in it. In place:
// on return every rank's copy holds the sum. BF16: elements are bf16 (summed in fp32), else fp32.
template <bool BF16>
__global__ void __launch_bounds__(512)
nvls_allreduce_kernel(char* mc, long long nvec, NvlsPeers P) {
  uint32_t* mine = P.flags[P.rank];
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(mine + 2) + 1u;
  if (blockIdx.x == 0) {
    // this rank's input is complete (it was written by earlier work on this stream)
    if (threadIdx.x < P.world) {
      __threadfence_system();
      red_release_sys_add(P.flags[threadIdx.x] + 0, 1u);
    }
    if (threadIdx.x == 0) {
      if (!wait_flag_ge(mine + 0, uint32_t(P.world) * call)) atomicExch(&g_nvls_status, kStatusPeerTimeout);
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(mine + 4) = call;      // open the gate for the other blocks
    }
  } else if (threadIdx.x == 0) {
    if (!wait_flag_ge(mine + 4, call)) atomicExch(&g_nvls_status, kStatusPeerTimeout);
  }
  __syncthreads();
  // this rank's slice, four vectors in flight per thread
  const long long per_rank = (nvec + P.world - 1) / P.world;
  const long long lo = per_rank * P.rank, hi = min(nvec, lo + per_rank);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j * stride < hi) v[j] = BF16 ? mm_ld_reduce_bf16(mc + (i + j * stride) * 16) : mm_ld_reduce_f32(mc + (i + j * stride) * 16);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i + j * stride < hi) mm_st(mc + (i + j * stride) * 16, v[j]);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(mine + 3, 1u) == gridDim.x - 1) {
      // last block of this rank: the whole slice is in every rank's copy
      mine[3] = 0u;
      __threadfence_system();
      for (int p = 0; p < P.world; ++p) red_release_sys_add(P.flags[p] + 1, 1u);
      if (!wait_flag_ge(mine + 1, uint32_t(P.world) * call)) atomicExch(&g_nvls_status, kStatusPeerTimeout);
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(mine + 2) = call;
    }
  }
}

}  // namespace rb

using namespace rb;

extern "C" int rmlx_nvls_flag_bytes() { return kNvlsFlagWords * 4; }

extern "C" int rmlx_nvls_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_nvls_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_nvls_status, &zero, sizeof(int));
  return v;
}

// mc: multicast address of the operand; bytes: multiple of 16; flags: host array of `world` device
// pointers to the ranks' flag areas (zero-initialised, rmlx_nvls_flag_bytes() each); blocks: grid
// size (1..64; 0 = chosen from the size). The grid must be resident at once (it is far below the
// number of SMs): blocks other than the first wait for a gate that the first one opens.
extern "C" int rmlx_nvls_allreduce(void* mc, long long bytes, int bf16, void* const* flags, int rank,
                                   int world, int blocks, cudaStream_t st) {
  if (!mc || bytes < 16 || bytes % 16 || (reinterpret_cast<uintptr_t>(mc) & 15u) || world < 1 ||
      world > kNvlsMaxWorld || rank < 0 || rank >= world)
    return -2;
  NvlsPeers P;
  for (int i = 0; i < kNvlsMaxWorld; ++i) P.flags[i] = i < world ? static_cast<uint32_t*>(flags[i]) : nullptr;
  P.rank = rank; P.world = world;
  const long long nvec = bytes / 16;
  if (blocks < 0 || blocks > kNvlsMaxBlocks) return -2;
  if (blocks == 0) {
    const long long per_rank = (nvec + world - 1) / world;
    blocks = int((per_rank + 4 * 512 - 1) / (4 * 512));
    if (blocks < 1) blocks = 1;
    if (blocks > kNvlsMaxBlocks) blocks = kNvlsMaxBlocks;
  }
  if (bf16) nvls_allreduce_kernel<true><<<blocks, 512, 0, st>>>(static_cast<char*>(mc), nvec, P);
  else nvls_allreduce_kernel<false><<<blocks, 512, 0, st>>>(static_cast<char*>(mc), nvec, P);
  return static_cast<int>(cudaGetLastError());
}
