// Host-side launch helpers shared by every kernel file: error propagation as plain ints (the
// Python side raises), dynamic shared-memory opt-in, SM count, and launches that can carry the
// programmatic-dependent-launch attribute so consecutive decode kernels overlap their prologues.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef RMLX_BOUNDS
#include <vector>
#endif

namespace rb {

// Bounds-checked build: every source file that uses RB_BOUNDS registers a reader of its own
// record (RB_BOUNDS_REGISTER at file scope); rmlx_bounds_status() walks the list.
#ifdef RMLX_BOUNDS
struct BoundsSource { const char* file; int (*read)(int* out4, int clear); };
inline std::vector<BoundsSource>& bounds_sources() { static std::vector<BoundsSource> v; return v; }
#define RB_BOUNDS_REGISTER(name)                                                                   \
  static int rb_bounds_read(int* out4, int clear) {                                                \
    if (cudaMemcpyFromSymbol(out4, ::rb::g_rb_bounds, 16) != cudaSuccess) return -1;               \
    if (clear && out4[0]) { const int z[4] = {0, 0, 0, 0}; (void)cudaMemcpyToSymbol(::rb::g_rb_bounds, z, 16); } \
    return 0;                                                                                      \
  }                                                                                                \
  static const bool rb_bounds_registered = (::rb::bounds_sources().push_back({name, rb_bounds_read}), true);
#else
#define RB_BOUNDS_REGISTER(name)
#endif

#define RB_CHECK(expr)                                   \
  do {                                                   \
    cudaError_t _e = (expr);                             \
    if (_e != cudaSuccess) return static_cast<int>(_e);  \
  } while (0)

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Opt in to more than 48 KB of dynamic shared memory. The attribute is per function per device;
// setting it again is cheap and legal during stream capture (it is not a stream operation).
template <class Kern>
inline cudaError_t set_max_smem(Kern kern, size_t bytes) {
  // the 48 KB default limit counts static shared memory too: opt in well below it
  if (bytes <= 24 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(bytes));
}

// Ask for the largest shared-memory carve-out. The kernels of a decode step are chained with
// programmatic dependent launch; an SM whose L1 / shared-memory split has to change between two
// kernels must drain first, which would undo the overlap, so every kernel of the chain asks for
// the same split.
template <class Kern>
inline void prefer_max_shared(Kern kern) {
  (void)cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
}

template <class... KArgs, class... Args>
inline int launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                  bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  if (pdl) prefer_max_shared(kern);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) (void)cudaGetLastError();  // do not leave a stale launch error behind
  return static_cast<int>(e);
}

}  // namespace rb
