// All-reduce done by the NVLink switch: the operands sit at the same offset of the symmetric heap
// on every rank, the heap segment is bound to a multicast object, and each rank reduces its own
// slice with `multimem.ld_reduce` (the switch fetches the slice from every rank and returns the
// sum) and writes it back with `multimem.st` (the switch stores it into every rank's copy). Two
// crossings of the fabric per element, no rank reads another rank's memory with ordinary loads.
//
// Counterpart of the reference's ring / tree all-reduce over RDMA
// (crates/rmlx-distributed/src/group.rs:348-504), which has no in-fabric reduction to use.
//
// Flags: block b of every rank signals word b of every rank's flag area (plain peer mappings,
// release adds) when this rank's input is complete, and again when its slice has been broadcast.
// Counters only grow: the call number lives in the flag area (word 2 * kMaxBlocks), is read by
// every block at its start and advanced by the last block to leave, so captured and eager calls
// can be mixed. Every wait is bounded and reports through a status word.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"

namespace rb {

constexpr int kNvlsMaxWorld = 8;
constexpr int kNvlsMaxBlocks = 64;
// flag area (u32 words): [0, 64) input-ready counters, [64, 128) done counters, 128 call number,
// 129 exit ticket, 130 grid size of the first call. Block b counts on word b, so every call on one
// flag area must use the same number of blocks (a block index that sat out a call would fall
// behind the call number); the kernel checks it and refuses a different grid.
constexpr int kNvlsFlagWords = 2 * kNvlsMaxBlocks + 3;

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
  const uint32_t g0 = atomicCAS(mine + 2 * kNvlsMaxBlocks + 2, 0u, gridDim.x);
  if (g0 != 0u && g0 != gridDim.x) {         // uniform over the grid: every block sees the same word
    if (threadIdx.x == 0) atomicExch(&g_nvls_status, kStatusBadArgument);
    return;
  }
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(mine + 2 * kNvlsMaxBlocks) + 1u;
  const int b = blockIdx.x;
  // this rank's input is complete (it was written by earlier work on this stream)
  if (threadIdx.x < P.world) {
    __threadfence_system();
    red_release_sys_add(P.flags[threadIdx.x] + b, 1u);
  }
  if (threadIdx.x == 0) {
    if (!wait_flag_ge(mine + b, uint32_t(P.world) * call)) atomicExch(&g_nvls_status, kStatusPeerTimeout);
  }
  __syncthreads();
  // this rank's slice, cut into gridDim.x parts
  const long long per_rank = (nvec + P.world - 1) / P.world;
  const long long lo = per_rank * P.rank, hi = min(nvec, lo + per_rank);
  for (long long i = lo + (long long)b * blockDim.x + threadIdx.x; i < hi; i += (long long)gridDim.x * blockDim.x) {
    char* p = mc + i * 16;
    const uint4 v = BF16 ? mm_ld_reduce_bf16(p) : mm_ld_reduce_f32(p);
    mm_st(p, v);
  }
  __syncthreads();
  // this block's part of the slice is in every rank's copy
  if (threadIdx.x < P.world) {
    __threadfence_system();
    red_release_sys_add(P.flags[threadIdx.x] + kNvlsMaxBlocks + b, 1u);
  }
  if (threadIdx.x == 0) {
    if (!wait_flag_ge(mine + kNvlsMaxBlocks + b, uint32_t(P.world) * call))
      atomicExch(&g_nvls_status, kStatusPeerTimeout);
    __threadfence();
    uint32_t* ticket = mine + 2 * kNvlsMaxBlocks + 1;
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(mine + 2 * kNvlsMaxBlocks) = call;
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
// size, the same on every call that uses these flag areas (1..64).
extern "C" int rmlx_nvls_allreduce(void* mc, long long bytes, int bf16, void* const* flags, int rank,
                                   int world, int blocks, cudaStream_t st) {
  if (!mc || bytes < 16 || bytes % 16 || (reinterpret_cast<uintptr_t>(mc) & 15u) || world < 1 ||
      world > kNvlsMaxWorld || rank < 0 || rank >= world)
    return -2;
  NvlsPeers P;
  for (int i = 0; i < kNvlsMaxWorld; ++i) P.flags[i] = i < world ? static_cast<uint32_t*>(flags[i]) : nullptr;
  P.rank = rank; P.world = world;
  const long long nvec = bytes / 16;
  if (blocks < 1 || blocks > kNvlsMaxBlocks) return -2;
  if (bf16) nvls_allreduce_kernel<true><<<blocks, 512, 0, st>>>(static_cast<char*>(mc), nvec, P);
  else nvls_allreduce_kernel<false><<<blocks, 512, 0, st>>>(static_cast<char*>(mc), nvec, P);
  return static_cast<int>(cudaGetLastError());
}
