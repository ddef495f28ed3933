// Small memory-bound kernels around the hot path: embedding gather, stand-alone RMSNorm (with the
// residual-add form), greedy arg-max over logits, SwiGLU elementwise, and per-token FP8 (E4M3)
// quantise/dequantise used by the optional FP8 expert-dispatch payload.
//
// Counterparts: crates/rmlx-nn/src/embedding.rs:60, crates/rmlx-core/src/ops/rms_norm.rs:86-807,
// crates/rmlx-core/src/ops/argreduce.rs, crates/rmlx-core/src/ops/silu.rs,
// crates/rmlx-core/src/ops/fp8.rs:55-378.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"
#include <cuda_fp8.h>

namespace rb {

__global__ void embedding_kernel(const __nv_bfloat16* __restrict__ table,
                                 const int* __restrict__ ids, __nv_bfloat16* __restrict__ out,
                                 int D, int vocab) {
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  int id = ids[blockIdx.x];
  (void)RB_BOUNDS(id, vocab);               // bounds-checked build: record it; the clamp keeps the read safe
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + size_t(id) * D);
  uint4* dst = reinterpret_cast<uint4*>(out + size_t(blockIdx.x) * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
  pdl_launch_dependents();
}

// out = rmsnorm(x (+ residual)) * w ; when residual is given, sum_out (may alias x) gets x+residual.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                __nv_bfloat16* __restrict__ sum_out, int D, float eps) {
  __shared__ float red[8];
  __shared__ float s_inv;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const size_t base = size_t(blockIdx.x) * D;
  float ssq = 0.f;
  for (int i = threadIdx.x; i < D; i += 256) {
    float v = __bfloat162float(x[base + i]);
    if (residual) {
      v += __bfloat162float(residual[base + i]);
      v = __bfloat162float(__float2bfloat16_rn(v));
      if (sum_out) sum_out[base + i] = __float2bfloat16_rn(v);
    }
    ssq += v * v;
  }
  ssq = warp_sum(ssq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) s_inv = rsqrtf(t / float(D) + eps);
  }
  __syncthreads();
  const float inv = s_inv;
  for (int i = threadIdx.x; i < D; i += 256) {
    float v = residual ? __bfloat162float(sum_out ? sum_out[base + i]
                                                  : __float2bfloat16_rn(__bfloat162float(x[base + i]) +
                                                                        __bfloat162float(residual[base + i])))
                       : __bfloat162float(x[base + i]);
    out[base + i] = __float2bfloat16_rn(v * inv * (w ? __bfloat162float(w[i]) : 1.f));
  }
  pdl_launch_dependents();
}

// Index of the row maximum (lowest index on ties). grid = (slices, rows): every block reduces its
// slice to one 64-bit key (order-preserving float bits, then inverted index), merges it with
// atomicMax, and the last block of a row decodes the winner and clears the scratch for the next
// launch. keys[rows] and tickets[rows] must be zero on first use.
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V, int stride,
              unsigned long long* __restrict__ keys, unsigned int* __restrict__ tickets) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const float* row = logits + size_t(blockIdx.y) * stride;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = blockIdx.x * 1024 + threadIdx.x; i < V; i += gridDim.x * 1024) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = sv[threadIdx.x]; bi = si[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (threadIdx.x == 0) {
      uint32_t u = __float_as_uint(best);
      u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;          // monotone map float -> uint
      const unsigned long long key =
          (static_cast<unsigned long long>(u) << 32) | (0xffffffffu - static_cast<uint32_t>(bi));
      atomicMax(keys + blockIdx.y, key);
      __threadfence();
      if (atomicAdd(tickets + blockIdx.y, 1u) == gridDim.x - 1) {
        __threadfence();
        const unsigned long long k = atomicExch(keys + blockIdx.y, 0ull);
        out[blockIdx.y] = static_cast<int>(0xffffffffu - static_cast<uint32_t>(k & 0xffffffffull));
        tickets[blockIdx.y] = 0u;
      }
    }
  }
  pdl_launch_dependents();
}

// act[t, i] = silu(gu[t, i]) * gu[t, I + i]
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                long long total, int I) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / I;
  const int i = int(idx % I);
  const float g = __bfloat162float(gu[t * 2 * I + i]), u = __bfloat162float(gu[t * 2 * I + I + i]);
  const float e = __expf(-fabsf(g));
  const float sig = g >= 0.f ? 1.f / (1.f + e) : e / (1.f + e);
  act[idx] = __float2bfloat16_rn(g * sig * u);
}

// Per-token E4M3 quantisation: scale = max|x| / 448 (crates/rmlx-distributed/src/fp8_exchange.rs:85-160).
__global__ void __launch_bounds__(256)
fp8_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_storage_t* __restrict__ q,
                      float* __restrict__ scales, int D) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const size_t base = size_t(blockIdx.x) * D;
  float m = 0.f;
  for (int i = threadIdx.x; i < D; i += 256) m = fmaxf(m, fabsf(__bfloat162float(x[base + i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_max(t);
    if (threadIdx.x == 0) { s_scale = t > 0.f ? t / 448.f : 1.f; scales[blockIdx.x] = s_scale; }
  }
  __syncthreads();
  const float inv = 1.f / s_scale;
  for (int i = threadIdx.x; i < D; i += 256)
    q[base + i] = __nv_cvt_float_to_fp8(__bfloat162float(x[base + i]) * inv, __NV_SATFINITE, __NV_E4M3);
}

__global__ void fp8_dequant_rows_kernel(const __nv_fp8_storage_t* __restrict__ q,
                                        const float* __restrict__ scales,
                                        __nv_bfloat16* __restrict__ out, int D) {
  const size_t base = size_t(blockIdx.x) * D;
  const float s = scales[blockIdx.x];
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(q[base + i], __NV_E4M3);
    out[base + i] = __float2bfloat16_rn(__half2float(*reinterpret_cast<const __half*>(&h)) * s);
  }
}

// End of a decode step: the sampled token becomes the next input and the sequence grows by one.
// Running this inside the captured step keeps the host out of the token loop.
__global__ void decode_advance_kernel(const int* __restrict__ next, int* __restrict__ tokens,
                                      int* __restrict__ positions, int* __restrict__ seq_lens,
                                      const int* __restrict__ active, int B) {
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B && (!active || active[b])) {
    tokens[b] = next[b];
    positions[b] += 1;
    seq_lens[b] += 1;
  }
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("misc.cu")


extern "C" int rmlx_decode_advance(const int* next, int* tokens, int* positions, int* seq_lens,
                                   const int* active, int B, int pdl, cudaStream_t st) {
  if (B < 1) return -2;
  return launch(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, st, pdl != 0, next,
                tokens, positions, seq_lens, active, B);
}

extern "C" const char* rmlx_error_string(int code) {
  return cudaGetErrorString(static_cast<cudaError_t>(code));
}

extern "C" int rmlx_embedding(const void* table, const int* ids, void* out, int T, int D, int vocab,
                              int pdl, cudaStream_t st) {
  if (T < 1 || D % 8) return -2;
  return launch(embedding_kernel, dim3(T), dim3(128), 0, st, pdl != 0,
                static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), D,
                vocab);
}

extern "C" int rmlx_rms_norm(const void* x, const void* residual, const void* w, void* out,
                             void* sum_out, int T, int D, float eps, int pdl, cudaStream_t st) {
  if (T < 1) return -2;
  return launch(rms_norm_kernel, dim3(T), dim3(256), 0, st, pdl != 0,
                static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
                static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(out),
                static_cast<__nv_bfloat16*>(sum_out), D, eps);
}

extern "C" int rmlx_argmax(const float* logits, int* out, int B, int V, int stride,
                           unsigned long long* keys, unsigned int* tickets, int pdl,
                           cudaStream_t st) {
  if (B < 1 || V < 1 || !keys || !tickets) return -2;
  int slices = (V + 4095) / 4096;
  if (slices > 64) slices = 64;
  return launch(argmax_kernel, dim3(slices, B), dim3(1024), 0, st, pdl != 0, logits, out, V, stride,
                keys, tickets);
}

extern "C" int rmlx_silu_mul(const void* gate_up, void* act, long long T, int I, cudaStream_t st) {
  const long long total = T * I;
  if (total < 1) return -2;
  silu_mul_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(act), total, I);
  return static_cast<int>(cudaGetLastError());
}

// Affine group-64 dequantisation to bf16: w = scale * q + bias, q packed little-endian in 32-bit
// words (4 or 8 bits per value). One thread per packed word. The prompt path expands 8-bit weights
// this way before its bf16 tensor-core GEMM (the 4-bit weights are expanded inside the GEMM).
// Reference: dequantize rows of affine_qmm (crates/rmlx-core/src/ops/quantized.rs:2755).
template <int BITS, bool SF16>
__global__ void __launch_bounds__(256)
dequant_affine_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                      const uint16_t* __restrict__ biases, __nv_bfloat16* __restrict__ out,
                      long long words, int K) {
  constexpr int PER = 32 / BITS;
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= words) return;
  const int wpr = K / PER;                       // words per row
  const long long row = i / wpr;
  const int col = int(i - row * wpr) * PER;
  const long long g = row * (K / 64) + col / 64;
  const float sc = SF16 ? __half2float(__ushort_as_half(scales[g])) : bf16lo(scales[g]);
  const float bi = SF16 ? __half2float(__ushort_as_half(biases[g])) : bf16lo(biases[g]);
  const uint32_t v = w[i];
  __nv_bfloat16* o = out + row * K + col;
#pragma unroll
  for (int j = 0; j < PER; j += 2) {
    const float a = float((v >> (j * BITS)) & ((1u << BITS) - 1u)) * sc + bi;
    const float b = float((v >> ((j + 1) * BITS)) & ((1u << BITS) - 1u)) * sc + bi;
    *reinterpret_cast<uint32_t*>(o + j) = pack_bf16(a, b);
  }
}

// w: packed words of `rows` x K values (bits 4 or 8), scales / biases [rows, K/64] in bf16 or
// (scale_f16) fp16, out bf16.
extern "C" int rmlx_dequant_affine(const void* w, const void* scales, const void* biases, void* out,
                                   long long rows, int K, int bits, int scale_f16, cudaStream_t st) {
  if (rows < 1 || K % 64 || (bits != 4 && bits != 8)) return -2;
  const long long words = rows * (K / (32 / bits));
  const unsigned grid = unsigned((words + 255) / 256);
#define RB_DQ(BITS_, SF_)                                                                         \
  dequant_affine_kernel<BITS_, SF_><<<grid, 256, 0, st>>>(                                        \
      static_cast<const uint32_t*>(w), static_cast<const uint16_t*>(scales),                      \
      static_cast<const uint16_t*>(biases), static_cast<__nv_bfloat16*>(out), words, K)
  if (bits == 4) { if (scale_f16) RB_DQ(4, true); else RB_DQ(4, false); }
  else { if (scale_f16) RB_DQ(8, true); else RB_DQ(8, false); }
#undef RB_DQ
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_fp8_quant_rows(const void* x, void* q, float* scales, int T, int D,
                                   cudaStream_t st) {
  if (T < 1) return -2;
  fp8_quant_rows_kernel<<<T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                           static_cast<__nv_fp8_storage_t*>(q), scales, D);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_fp8_dequant_rows(const void* q, const float* scales, void* out, int T, int D,
                                     cudaStream_t st) {
  if (T < 1) return -2;
  fp8_dequant_rows_kernel<<<T, 256, 0, st>>>(static_cast<const __nv_fp8_storage_t*>(q), scales,
                                             static_cast<__nv_bfloat16*>(out), D);
  return static_cast<int>(cudaGetLastError());
}

// ---- bounds-checked build ---------------------------------------------------------------------
// 1 when this library was compiled with -DRMLX_BOUNDS.
extern "C" int rmlx_bounds_build() {
#ifdef RMLX_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Reads (and clears) the first recorded out-of-range index: out4 = {status code, source line,
// index, limit}, `file` the source file that recorded it. Returns 1 when a record was found, 0 when
// none, -1 on a runtime error, -3 when this is not a bounds-checked build.
extern "C" int rmlx_bounds_status(int* out4, char* file, int file_len) {
#ifdef RMLX_BOUNDS
  for (const auto& src : bounds_sources()) {
    int rec[4] = {0, 0, 0, 0};
    if (src.read(rec, 1) != 0) return -1;
    if (rec[0]) {
      for (int i = 0; i < 4; ++i) out4[i] = rec[i];
      if (file && file_len > 0) {
        int i = 0;
        for (; src.file[i] && i < file_len - 1; ++i) file[i] = src.file[i];
        file[i] = 0;
      }
      return 1;
    }
  }
  return 0;
#else
  (void)out4; (void)file; (void)file_len;
  return -3;
#endif
}

// ---- AWQ / GPTQ 4-bit checkpoints -> fp32 [out, in] (exact: a small integer times an fp16) ------
// AWQ: qweight int32 [in, out/8], qzeros int32 [in/g, out/8], scales fp16 [in/g, out]; logical
// output j of a word is nibble {0, 4, 1, 5, 2, 6, 3, 7}[j]; w = (q - z) * s
// (crates/rmlx-core/src/ops/quantized.rs:707, awq_dequant_f32).
// GPTQ: qweight int32 [in/8, out] (nibble j of a word is input 8*iw + j), qzeros int32
// [groups, out/8] (stored zero + 1 is the zero point), scales fp16 [groups, out], g_idx [in] (or
// null: consecutive groups); w = (q - (z + 1)) * s (quantized.rs:749, gptq_dequant_f32).
namespace rb {

__global__ void __launch_bounds__(256)
awq_dequant_kernel(const uint32_t* __restrict__ qweight, const uint32_t* __restrict__ qzeros,
                   const __half* __restrict__ scales, float* __restrict__ out, int in_f,
                   int out_f, int group) {
  const int out8 = out_f >> 3;
  const long long idx = blockIdx.x * 256LL + threadIdx.x;      // (ob, i): i fastest -> coalesced stores
  if (idx >= 1LL * in_f * out8) return;
  const int i = int(idx % in_f), ob = int(idx / in_f);
  const int g = i / group;
  const uint32_t w = qweight[size_t(i) * out8 + ob], z = qzeros[size_t(g) * out8 + ob];
  const int order[8] = {0, 4, 1, 5, 2, 6, 3, 7};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int q = int((w >> (4 * order[j])) & 0xFu) - int((z >> (4 * order[j])) & 0xFu);
    const float s = __half2float(scales[size_t(g) * out_f + ob * 8 + j]);
    out[size_t(ob * 8 + j) * in_f + i] = float(q) * s;
  }
}

__global__ void __launch_bounds__(256)
gptq_dequant_kernel(const uint32_t* __restrict__ qweight, const uint32_t* __restrict__ qzeros,
                    const __half* __restrict__ scales, const int* __restrict__ g_idx,
                    float* __restrict__ out, int in_f, int out_f, int groups) {
  const int in8 = in_f >> 3, out8 = out_f >> 3;
  const long long idx = blockIdx.x * 256LL + threadIdx.x;      // (iw, o): o fastest -> coalesced loads
  if (idx >= 1LL * in8 * out_f) return;
  const int o = int(idx % out_f), iw = int(idx / out_f);
  const uint32_t w = qweight[size_t(iw) * out_f + o];
  const int per_group = in_f / groups;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = iw * 8 + j;
    const int g = g_idx ? g_idx[i] : i / per_group;
    const int z = int((qzeros[size_t(g) * out8 + (o >> 3)] >> (4 * (o & 7))) & 0xFu) + 1;
    v[j] = float(int((w >> (4 * j)) & 0xFu) - z) * __half2float(scales[size_t(g) * out_f + o]);
  }
  float4* dst = reinterpret_cast<float4*>(out + size_t(o) * in_f + iw * 8);
  dst[0] = make_float4(v[0], v[1], v[2], v[3]);
  dst[1] = make_float4(v[4], v[5], v[6], v[7]);
}

}  // namespace rb

extern "C" int rmlx_awq_dequant(const void* qweight, const void* qzeros, const void* scales, void* out,
                                int in_f, int out_f, int group, cudaStream_t st) {
  if (in_f < 1 || out_f < 8 || out_f % 8 || group < 1 || in_f % group) return -2;
  const long long n = 1LL * in_f * (out_f / 8);
  rb::awq_dequant_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(
      static_cast<const uint32_t*>(qweight), static_cast<const uint32_t*>(qzeros),
      static_cast<const __half*>(scales), static_cast<float*>(out), in_f, out_f, group);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_gptq_dequant(const void* qweight, const void* qzeros, const void* scales,
                                 const int* g_idx, void* out, int in_f, int out_f, int groups,
                                 cudaStream_t st) {
  if (in_f < 8 || in_f % 8 || out_f < 8 || out_f % 8 || groups < 1 || in_f % groups) return -2;
  const long long n = 1LL * (in_f / 8) * out_f;
  rb::gptq_dequant_kernel<<<unsigned((n + 255) / 256), 256, 0, st>>>(
      static_cast<const uint32_t*>(qweight), static_cast<const uint32_t*>(qzeros),
      static_cast<const __half*>(scales), g_idx, static_cast<float*>(out), in_f, out_f, groups);
  return static_cast<int>(cudaGetLastError());
}
