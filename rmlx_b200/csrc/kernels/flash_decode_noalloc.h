// Paged flash-decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework; it exists for embedders of this
// library that run where the CUDA allocator is off limits: inside a host that owns every byte of
// device memory and hands out none at run time, inside a real-time loop that may not take the
// allocator's locks, or from a plug-in interface that only passes input and output buffers. The
// regular entry point (rmlx_flash_decode_paged) needs three scratch buffers from its caller when
// the context is split across thread blocks; this one carries them itself, in a fixed array
// compiled into the library's device image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch covers: batch * kv_heads * ceil((q_heads/kv_heads)/16) tiles,
// KV splits per tile, and head dimension. The scratch array is ~8.2 MB and stays resident on every
// GPU that loads the library until the process exits.
#define RMLX_FD_NOALLOC_MAX_TILES 64
#define RMLX_FD_NOALLOC_MAX_SPLITS 16
#define RMLX_FD_NOALLOC_MAX_HEAD_DIM 128

// Error codes specific to this entry point (others are cudaError_t values, or -2 for an argument
// the regular entry point also rejects).
#define RMLX_FD_NOALLOC_TOO_LARGE (-5)    /* shape exceeds the limits above */
#define RMLX_FD_NOALLOC_SETUP_FAILED (-6) /* the device address of the scratch could not be resolved */

// Same arguments and result as rmlx_flash_decode_paged without the three scratch pointers.
// Calls no cudaMalloc / cudaFree and no allocating library routine.
//
// * The first call on each device resolves the scratch array's device address (once per device,
//   with that device current). Make that first call outside any stream capture.
// * The device that owns `stream` must be the current device of the calling thread: the scratch
//   address is looked up for the current device, not for the stream's. The first-call lookup is
//   not synchronised between host threads (concurrent first calls on one device all store the
//   same address, which is harmless, but do not rely on it for ordering).
// * All calls share the one scratch array, and it keeps whatever the previous call left in it
//   (the part that must start at zero, the per-tile tickets, is cleared on the stream by every
//   call). Two calls that overlap on the GPU, e.g. on different streams, race on it: serialise them.
int rmlx_flash_decode_paged_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                    const int* block_table, const int* seq_lens, void* out, int B,
                                    int Hq, int Hkv, int HD, int max_blocks, int splits, int window,
                                    float scale, cudaStream_t stream);

// Human-readable text for the codes above (NULL for other values).
const char* rmlx_flash_decode_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
