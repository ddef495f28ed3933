// Block dequantisers for the GGML tensor types found in GGUF checkpoints: F16, BF16, Q4_0, Q4_1,
// Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K and Q6_K to fp32, split over threads by blocks. The
// arithmetic follows the block layouts of the format (d * q with 4/5/8-bit quants and fp16 scales
// for the simple types; packed 4- or 6-bit sub-block scales and minima for Q2_K / Q4_K / Q5_K;
// signed 6-bit sub-block scales for Q3_K; 6-bit quants with int8 sub-block scales for Q6_K) in the
// same operation order as the numpy restatement in loader/gguf.py, so the two agree bit for bit
// and the Python one serves as the oracle.
//
// Native counterpart of the reference's CPU dequantisation of K-quants and legacy GGML types
// (crates/rmlx-nn/src/quantized_linear.rs:806 `KQuantConfig::dequantize_to_f32`,
// crates/rmlx-core/src/formats/gguf.rs).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {                                   // subnormal: renormalise
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      bits = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;     // inf / nan
  } else {
    bits = sign | (exp + 112u) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline float rd_f16(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return f16_to_f32(h);
}

// ggml type ids
enum : int { kF32 = 0, kF16 = 1, kQ4_0 = 2, kQ4_1 = 3, kQ5_0 = 6, kQ5_1 = 7, kQ8_0 = 8, kQ2_K = 10,
              kQ3_K = 11, kQ4_K = 12, kQ5_K = 13, kQ6_K = 14, kBF16 = 30 };

struct TypeInfo { int elems, bytes; };
bool type_info(int t, TypeInfo* out) {
  switch (t) {
    case kF32: *out = {1, 4}; return true;
    case kF16: *out = {1, 2}; return true;
    case kBF16: *out = {1, 2}; return true;
    case kQ4_0: *out = {32, 18}; return true;
    case kQ4_1: *out = {32, 20}; return true;
    case kQ5_0: *out = {32, 22}; return true;
    case kQ5_1: *out = {32, 24}; return true;
    case kQ8_0: *out = {32, 34}; return true;
    case kQ2_K: *out = {256, 84}; return true;
    case kQ3_K: *out = {256, 110}; return true;
    case kQ5_K: *out = {256, 176}; return true;
    case kQ4_K: *out = {256, 144}; return true;
    case kQ6_K: *out = {256, 210}; return true;
    default: return false;
  }
}

void block(int type, const uint8_t* b, float* o) {
  switch (type) {
    case kF32: memcpy(o, b, 4); break;
    case kF16: *o = rd_f16(b); break;
    case kBF16: {
      uint16_t h;
      memcpy(&h, b, 2);
      const uint32_t bits = static_cast<uint32_t>(h) << 16;
      memcpy(o, &bits, 4);
      break;
    }
    case kQ4_0: {
      const float d = rd_f16(b);
      for (int i = 0; i < 16; ++i) {
        o[i] = static_cast<float>(static_cast<int>(b[2 + i] & 0xF) - 8) * d;
        o[16 + i] = static_cast<float>(static_cast<int>(b[2 + i] >> 4) - 8) * d;
      }
      break;
    }
    case kQ4_1: {
      const float d = rd_f16(b), m = rd_f16(b + 2);
      for (int i = 0; i < 16; ++i) {
        o[i] = static_cast<float>(b[4 + i] & 0xF) * d + m;
        o[16 + i] = static_cast<float>(b[4 + i] >> 4) * d + m;
      }
      break;
    }
    case kQ8_0: {
      const float d = rd_f16(b);
      for (int i = 0; i < 32; ++i) o[i] = static_cast<float>(static_cast<int8_t>(b[2 + i])) * d;
      break;
    }
    case kQ5_0:
    case kQ5_1: {
      const int off = type == kQ5_0 ? 2 : 4;
      const float d = rd_f16(b), m = type == kQ5_1 ? rd_f16(b + 2) : 0.f;
      uint32_t qh;
      memcpy(&qh, b + off, 4);                 // bit j: fifth bit of value j
      const uint8_t* qs = b + off + 4;
      for (int i = 0; i < 16; ++i) {
        const int lo = (qs[i] & 0xF) | (((qh >> i) & 1u) << 4);
        const int hi = (qs[i] >> 4) | (((qh >> (i + 16)) & 1u) << 4);
        if (type == kQ5_0) {
          o[i] = static_cast<float>(lo - 16) * d;
          o[16 + i] = static_cast<float>(hi - 16) * d;
        } else {
          o[i] = static_cast<float>(lo) * d + m;
          o[16 + i] = static_cast<float>(hi) * d + m;
        }
      }
      break;
    }
    case kQ2_K: {
      const uint8_t* sc = b;                   // sixteen bytes: 4-bit scale (low) and 4-bit minimum (high)
      const uint8_t* qs = b + 16;
      const float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
      for (int n = 0; n < 2; ++n)
        for (int j = 0; j < 4; ++j)
          for (int h = 0; h < 2; ++h) {
            const uint8_t s = sc[8 * n + 2 * j + h];
            const float dl = d * static_cast<float>(s & 0xF), ml = dmin * static_cast<float>(s >> 4);
            float* out = o + 128 * n + 32 * j + 16 * h;
            const uint8_t* q = qs + 32 * n + 16 * h;
            for (int i = 0; i < 16; ++i) out[i] = dl * static_cast<float>((q[i] >> (2 * j)) & 3) - ml;
          }
      break;
    }
    case kQ3_K: {
      const uint8_t* hm = b;                   // 32 bytes: bit (4n + j) of byte i = high bit of value
      const uint8_t* qs = b + 32;
      const uint8_t* sr = b + 96;              // twelve bytes holding sixteen 6-bit scales
      const float d = rd_f16(b + 108);
      float scales[16];
      for (int k = 0; k < 16; ++k) {
        const int lo = k < 8 ? (sr[k] & 0xF) : (sr[k - 8] >> 4);
        const int hi = (sr[8 + (k & 3)] >> (2 * (k >> 2))) & 3;
        scales[k] = static_cast<float>(static_cast<int8_t>(lo | (hi << 4))) - 32.f;
      }
      for (int n = 0; n < 2; ++n)
        for (int j = 0; j < 4; ++j)
          for (int h = 0; h < 2; ++h) {
            const float dl = d * scales[8 * n + 2 * j + h];
            float* out = o + 128 * n + 32 * j + 16 * h;
            for (int i = 0; i < 16; ++i) {
              const int idx = 16 * h + i;
              const int v = static_cast<int>((qs[32 * n + idx] >> (2 * j)) & 3) -
                            (((hm[idx] >> (4 * n + j)) & 1) ? 0 : 4);
              out[i] = dl * static_cast<float>(v);
            }
          }
      break;
    }
    case kQ5_K: {
      const float d = rd_f16(b), dmin = rd_f16(b + 2);
      const uint8_t* s = b + 4;
      const uint8_t* qh = b + 16;
      const uint8_t* qs = b + 48;
      float sc[8], mn[8];
      for (int j = 0; j < 8; ++j) {
        if (j < 4) {
          sc[j] = static_cast<float>(s[j] & 63);
          mn[j] = static_cast<float>(s[j + 4] & 63);
        } else {
          sc[j] = static_cast<float>((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
          mn[j] = static_cast<float>((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
        }
      }
      for (int j = 0; j < 4; ++j) {
        const float d0 = d * sc[2 * j], m0 = dmin * mn[2 * j];
        const float d1 = d * sc[2 * j + 1], m1 = dmin * mn[2 * j + 1];
        for (int i = 0; i < 32; ++i) {
          const uint8_t q = qs[32 * j + i];
          const int lo = (q & 0xF) + (((qh[i] >> (2 * j)) & 1) << 4);
          const int hi = (q >> 4) + (((qh[i] >> (2 * j + 1)) & 1) << 4);
          o[64 * j + i] = d0 * static_cast<float>(lo) - m0;
          o[64 * j + 32 + i] = d1 * static_cast<float>(hi) - m1;
        }
      }
      break;
    }
    case kQ4_K: {
      const float d = rd_f16(b), dmin = rd_f16(b + 2);
      const uint8_t* s = b + 4;                 // 12 bytes: eight 6-bit scales and eight 6-bit minima
      const uint8_t* qs = b + 16;
      float sc[8], mn[8];
      for (int j = 0; j < 8; ++j) {
        if (j < 4) {
          sc[j] = static_cast<float>(s[j] & 63);
          mn[j] = static_cast<float>(s[j + 4] & 63);
        } else {
          sc[j] = static_cast<float>((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
          mn[j] = static_cast<float>((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
        }
      }
      for (int j = 0; j < 4; ++j) {
        const float d0 = d * sc[2 * j], m0 = dmin * mn[2 * j];
        const float d1 = d * sc[2 * j + 1], m1 = dmin * mn[2 * j + 1];
        for (int i = 0; i < 32; ++i) {
          const uint8_t q = qs[32 * j + i];
          o[64 * j + i] = d0 * static_cast<float>(q & 0xF) - m0;
          o[64 * j + 32 + i] = d1 * static_cast<float>(q >> 4) - m1;
        }
      }
      break;
    }
    case kQ6_K: {
      const uint8_t* ql = b;
      const uint8_t* qh = b + 128;
      const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
      const float d = rd_f16(b + 208);
      for (int half = 0; half < 2; ++half) {
        const uint8_t* l = ql + 64 * half;
        const uint8_t* h = qh + 32 * half;
        const int8_t* s = sc + 8 * half;
        float* out = o + 128 * half;
        for (int i = 0; i < 32; ++i) {
          const int g = i / 16;
          const int q1 = static_cast<int>((l[i] & 0xF) | (((h[i] >> 0) & 3) << 4)) - 32;
          const int q2 = static_cast<int>((l[32 + i] & 0xF) | (((h[i] >> 2) & 3) << 4)) - 32;
          const int q3 = static_cast<int>((l[i] >> 4) | (((h[i] >> 4) & 3) << 4)) - 32;
          const int q4 = static_cast<int>((l[32 + i] >> 4) | (((h[i] >> 6) & 3) << 4)) - 32;
          out[i] = d * static_cast<float>(s[g]) * static_cast<float>(q1);
          out[32 + i] = d * static_cast<float>(s[g + 2]) * static_cast<float>(q2);
          out[64 + i] = d * static_cast<float>(s[g + 4]) * static_cast<float>(q3);
          out[96 + i] = d * static_cast<float>(s[g + 6]) * static_cast<float>(q4);
        }
      }
      break;
    }
  }
}

}  // namespace

extern "C" {

// Elements and bytes of one block of a GGML type; 0 when the type has no dequantiser here.
int rmlx_ggml_block_elems(int type) { TypeInfo t; return type_info(type, &t) ? t.elems : 0; }
int rmlx_ggml_block_bytes(int type) { TypeInfo t; return type_info(type, &t) ? t.bytes : 0; }

// src: nblocks blocks of `type`; dst: nblocks * block_elems floats. threads 0 = choose.
// Returns 0, or -2 for an unknown type.
int rmlx_ggml_dequant(int type, const void* src, uint64_t nblocks, float* dst, int threads) {
  TypeInfo t;
  if (!type_info(type, &t)) return -2;
  const uint8_t* s = static_cast<const uint8_t*>(src);
  auto run = [=](uint64_t lo, uint64_t hi) {
    for (uint64_t i = lo; i < hi; ++i) block(type, s + i * t.bytes, dst + i * t.elems);
  };
  const uint64_t work = nblocks * static_cast<uint64_t>(t.elems);
  if (threads <= 0) threads = static_cast<int>(std::min<unsigned>(8, std::max<unsigned>(1, std::thread::hardware_concurrency())));
  const uint64_t kMin = 1u << 20;                          // elements per thread worth a thread
  const int n = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(static_cast<uint64_t>(threads), work / kMin)));
  if (n == 1) {
    run(0, nblocks);
    return 0;
  }
  std::vector<std::thread> pool;
  const uint64_t per = (nblocks + n - 1) / n;
  for (int k = 0; k < n; ++k) {
    const uint64_t lo = per * k, hi = std::min(nblocks, lo + per);
    if (lo >= hi) break;
    pool.emplace_back(run, lo, hi);
  }
  for (auto& th : pool) th.join();
  return 0;
}

}  // extern "C"
