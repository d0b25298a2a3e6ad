// Shared device helpers and host-side argument checks for the AWQ W4A16 kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "awq_b200.h"

namespace awq {

constexpr int kBlockK = 128;       // k-extent of one packed block: 16 words of 8 nibbles per column
constexpr int kWordsPerBlock = 16;

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return AWQ_B200_ERR_CUDA;
}

#define AWQ_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::awq::cuda_fail(_e);      \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Shape rules shared by every compute entry point.
inline int check_shape(int K, int N, int group_size) {
  if (K <= 0 || N <= 0 || K % kBlockK != 0 || N % 8 != 0) return AWQ_B200_ERR_SHAPE;
  if (group_size <= 0 || group_size % kBlockK != 0) return AWQ_B200_ERR_GROUP;
  if (K % group_size != 0) return AWQ_B200_ERR_SHAPE;
  return AWQ_B200_OK;
}

struct DeviceInfo {
  int sm_count;
  int cc_major;
  int max_smem_optin;
};
// Immutable properties of the current device, cached per device ordinal.
int device_info(DeviceInfo* out);

// ---------------------------------------------------------------------------
// device side: int4 -> fp16 dequantisation
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
  return r;
}

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));   // IEEE rn, subnormals kept
  return r;
}

// Per-(group, column) constants of the zero point, both halves equal.
struct ZeroPair {
  uint32_t lo;  // half2(1024 + z)
  uint32_t hi;  // half2(-(64 + z))
};
__device__ __forceinline__ ZeroPair make_zero_pair(uint32_t z) {
  ZeroPair p;
  p.lo = (0x6400u | z) * 0x00010001u;
  p.hi = (0xD400u | (z << 4)) * 0x00010001u;
  return p;
}

// Nibble position (within a qzeros / qweight word) of logical channel j = 0..7.
__device__ __forceinline__ uint32_t awq_slot_shift(uint32_t j) { return ((j >> 1) + ((j & 1u) << 2)) << 2; }

// One 32-bit word of 8 nibbles -> four half2 holding fp16(q - z) * s.
// Nibble i pairs with nibble i+4: out[i] = (nibble i, nibble i+4), i = 0..3.
// q - z is formed exactly: low nibbles as (1024+q) - (1024+z); nibbles in bits
// 4..7 as (1024+16q)/16 - (64+z) in one fma.  The only rounding is the final
// fp16 multiply by the scale, as in the reference's `(q - z) * s` on fp16
// tensors (LLMQRT/runtime_refact/utils/packing_utils.py:76-78).
__device__ __forceinline__ void dequant_word(uint32_t w, ZeroPair zp, uint32_t s2, uint32_t out[4]) {
  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u, kMagic = 0x64006400u;
  constexpr uint32_t kSixteenth = 0x2c002c00u;  // half2(1/16)
  const uint32_t w8 = w >> 8;
  const uint32_t a0 = lop3_and_or(w, kLoMask, kMagic);
  const uint32_t a1 = lop3_and_or(w, kHiMask, kMagic);
  const uint32_t a2 = lop3_and_or(w8, kLoMask, kMagic);
  const uint32_t a3 = lop3_and_or(w8, kHiMask, kMagic);
  out[0] = h2_mul(h2_sub(a0, zp.lo), s2);
  out[1] = h2_mul(h2_fma(a1, kSixteenth, zp.hi), s2);
  out[2] = h2_mul(h2_sub(a2, zp.lo), s2);
  out[3] = h2_mul(h2_fma(a3, kSixteenth, zp.hi), s2);
}

// Even split of U work units over G persistent CTAs (G <= U): CTA b owns units
// [stream_first_unit(b), stream_first_unit(b + 1)), and stream_cta_of(u) is the CTA that owns unit u.
__host__ __device__ inline long long stream_first_unit(long long b, long long U, long long G) { return b * U / G; }
__host__ __device__ inline int stream_cta_of(long long u, long long U, long long G) {
  return static_cast<int>(((u + 1) * G + U - 1) / U - 1);
}

__device__ __forceinline__ uint32_t half_bits_x2(uint16_t h) { return static_cast<uint32_t>(h) * 0x00010001u; }

#endif  // __CUDACC__

}  // namespace awq
