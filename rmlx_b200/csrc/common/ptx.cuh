// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor copies), tcgen05 (5th-gen tensor
// cores + tensor memory), programmatic dependent launch, and system-scope acquire/release accesses
// used for peer (NVLink) signalling.
//
// Every wait in this file is bounded: a spin gives up after a fixed number of polls and reports it,
// so a kernel can set an error status and leave instead of hanging a shared GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace rb {

// ----------------------------------------------------------------------------------------------
// Status word written by kernels when a bounded wait expires (host reads it after the launch).
// ----------------------------------------------------------------------------------------------
enum StatusCode : int {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,    // an mbarrier wait inside a pipelined kernel ran out
  kStatusPeerTimeout = 2,    // a wait on a flag written by another GPU ran out
  kStatusBadArgument = 3,    // device-side argument check failed (debug builds)
};

// Bounds-checked build (-DRMLX_BOUNDS, a second library beside the normal one): RB_BOUNDS(i, n)
// is true when 0 <= i < n; otherwise it records the first offender of this source file (code,
// source line, index, limit) in a device word the host reads with rmlx_bounds_status(), and the
// caller skips or redirects the access. In the normal build it is the constant true and costs
// nothing. This is the stand-in for a memory checker on boxes where none can run.
#ifdef RMLX_BOUNDS
static __device__ int g_rb_bounds[4];
__device__ __forceinline__ bool rb_in_bounds(long long i, long long n, int line) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_rb_bounds[0], 0, int(kStatusBadArgument)) == 0) {
    g_rb_bounds[1] = line;
    g_rb_bounds[2] = int(i);
    g_rb_bounds[3] = int(n);
  }
  return false;
}
#define RB_BOUNDS(i, n) ::rb::rb_in_bounds((long long)(i), (long long)(n), __LINE__)
#else
#define RB_BOUNDS(i, n) true
#endif

// Poll budgets. One poll of try_wait blocks for up to ~1-2 us in hardware, so 2^22 polls is a few
// seconds at worst; the peer-flag budget is counted in polls with a nanosleep between them.
constexpr uint32_t kMbarPollLimit = 1u << 22;
constexpr uint32_t kPeerPollLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------------------------
// Programmatic dependent launch. Both are no-ops when the kernel was launched without the
// programmatic-stream-serialization attribute.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. `abort_flag` is a CTA-shared word: once any role gives up, the others stop waiting
// at their next poll instead of each burning the full budget. Returns false on give-up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile uint32_t* abort_flag,
                                          uint32_t limit = kMbarPollLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u && *abort_flag) return false;
  }
  *abort_flag = 1u;
  return false;
}

// ----------------------------------------------------------------------------------------------
// TMA: tiled bulk tensor copies. Loads here never carry a cluster-broadcast qualifier: each CTA
// fetches its own tiles, which is the only form allowed in code that runs on more than one GPU.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* smem_src, int32_t x,
                                             int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: tensor memory allocation, MMA issue, commit, and accumulator read-back.
// ----------------------------------------------------------------------------------------------
// Executed by one full warp. `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the whole CTA.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread i of the warp receives row (lane base + i),
// columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The store counterpart: thread i of the warp writes row (lane base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major bf16 tile stored as rows of 128 bytes (64 bf16)
// with the 128-byte swizzle, eight-row groups 1024 bytes apart. `smem_addr` is 1024-byte aligned
// for the tile base; advancing along K inside the 128-byte row adds the byte offset to the start
// address (16 elements = 32 bytes per MMA of K = 16).
__device__ __forceinline__ uint64_t umma_desc_sw128_kmajor(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address  [0,14)
  d |= static_cast<uint64_t>(1u) << 16;                           // leading byte offset (unused)
  d |= static_cast<uint64_t>(1024u >> 4) << 32;                   // stride byte offset [32,46)
  d |= static_cast<uint64_t>(1u) << 46;                           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2u) << 61;                           // layout: 128-byte swizzle
  return d;
}
// Descriptor for an MN-major bf16 operand: rows are steps along K (one row = 64 consecutive
// elements of the M/N dimension = 128 bytes, 128-byte swizzle), eight-row groups 1024 bytes apart,
// and the next 64 elements of the M/N dimension start `mn_panel_bytes` further on. This is the
// shape in which a [keys, head_dim] value tile lands when TMA loads it as 64-column panels.
// Advancing along K by 8 rows adds 1024 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_sw128_mnmajor(uint32_t smem_addr,
                                                            uint32_t mn_panel_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address  [0,14)
  d |= static_cast<uint64_t>((mn_panel_bytes >> 4) & 0x3FFFu) << 16;  // leading byte offset
  d |= static_cast<uint64_t>(1024u >> 4) << 32;                   // stride byte offset [32,46)
  d |= static_cast<uint64_t>(1u) << 46;                           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2u) << 61;                           // layout: 128-byte swizzle
  return d;
}
// Bit 16 of the instruction descriptor: operand B is MN-major instead of K-major.
constexpr uint32_t kUmmaBMajorMN = 1u << 16;
// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), fp32 accumulate.
__host__ __device__ constexpr uint32_t umma_idesc_bf16_f32(int m, int n) {
  return (1u << 4)                               // D format: f32
         | (1u << 7)                             // A format: bf16
         | (1u << 10)                            // B format: bf16
         | (static_cast<uint32_t>(n >> 3) << 17) // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);// M / 16
}

// ----------------------------------------------------------------------------------------------
// System-scope signalling on peer-visible memory.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Wait until *p >= target (epochs only grow, so no reset race). Returns false after the budget.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target,
                                             uint32_t limit = kPeerPollLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return true;
    if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
  }
  return false;
}

// ----------------------------------------------------------------------------------------------
// Streaming global loads (weights are read once per step: keep them out of L1).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// bf16 pair packed in a 32-bit word -> two floats (exact: bf16 is the top half of an fp32).
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace rb
