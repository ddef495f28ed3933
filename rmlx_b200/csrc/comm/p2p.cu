// Point-to-point put / get over the symmetric heap: a copy kernel that moves bytes between this
// rank's memory and a peer's mapping (16-byte vectors, any number of blocks), and the two ends of
// a message handshake: `signal` adds to a counter in the receiver's memory after a system-scope
// fence, `wait` polls the local counter with a bound. Counters only grow (message k waits for k).
//
// This is the send / recv layer of the reference's RDMA connection (post_send / post_recv /
// wait_completion on a queue pair, crates/rmlx-rdma/src/connection.rs) on NVLink: a put is a
// kernel storing into the peer, a completion is a counter the peer reads.
#include "../common/launch.cuh"
#include "../common/ptx.cuh"

namespace rb {

__device__ int g_p2p_status = 0;

// dst / src: 16-byte aligned; n16: number of 16-byte vectors; tail bytes handled by thread 0.
__global__ void __launch_bounds__(256)
p2p_copy_kernel(char* __restrict__ dst, const char* __restrict__ src, long long n16, int tail,
                uint32_t* signal_word, uint32_t* ticket) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n16;
       i += (long long)gridDim.x * blockDim.x)
    d[i] = s[i];
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (int b = 0; b < tail; ++b) dst[n16 * 16 + b] = src[n16 * 16 + b];
  if (signal_word == nullptr) return;
  // the last block to finish publishes the message: every store above is ordered before the add
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence_system();
      red_release_sys_add(signal_word, 1u);
    }
  }
}

__global__ void p2p_signal_kernel(uint32_t* word, uint32_t amount) {
  __threadfence_system();
  red_release_sys_add(word, amount);
}

__global__ void p2p_wait_kernel(const uint32_t* word, uint32_t target, uint32_t limit) {
  if (!wait_flag_ge(word, target, limit)) atomicExch(&g_p2p_status, kStatusPeerTimeout);
}

}  // namespace rb

using namespace rb;

extern "C" int rmlx_p2p_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_p2p_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_p2p_status, &zero, sizeof(int));
  return v;
}

// Copy `bytes` from src to dst (either may be a peer mapping; both 16-byte aligned). With
// signal_word (an address in the RECEIVER's memory) the last block adds 1 to it once every byte has
// been stored; `ticket` is a zero-initialised local word used to find the last block.
extern "C" int rmlx_p2p_put(void* dst, const void* src, long long bytes, void* signal_word,
                            void* ticket, int blocks, cudaStream_t st) {
  if (bytes < 0 || (reinterpret_cast<uintptr_t>(dst) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u))
    return -2;
  if (signal_word && !ticket) return -2;
  if (blocks < 1) blocks = int(bytes / (256 * 16 * 8)) + 1;
  if (blocks > 128) blocks = 128;
  p2p_copy_kernel<<<blocks, 256, 0, st>>>(static_cast<char*>(dst), static_cast<const char*>(src),
                                           bytes / 16, int(bytes % 16),
                                           static_cast<uint32_t*>(signal_word),
                                           static_cast<uint32_t*>(ticket));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_p2p_signal(void* word, unsigned int amount, cudaStream_t st) {
  p2p_signal_kernel<<<1, 1, 0, st>>>(static_cast<uint32_t*>(word), amount);
  return static_cast<int>(cudaGetLastError());
}

// Wait on the stream until *word >= target; limit: polls (0 = the default bound). An expired wait
// sets the status word (rmlx_p2p_status) and the stream continues.
extern "C" int rmlx_p2p_wait(const void* word, unsigned int target, unsigned int limit, cudaStream_t st) {
  p2p_wait_kernel<<<1, 1, 0, st>>>(static_cast<const uint32_t*>(word), target,
                                   limit ? limit : kPeerPollLimit);
  return static_cast<int>(cudaGetLastError());
}
