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

// Shape rules shared by every compute entry point.  Group sizes: any multiple of 128, and 32 or 64 for the
// kernels that build the exact fp16 weight per element (`small_groups`: the tensor-memory GEMMs and the
// exact-weight split-K kernel); the decode kernels that rescale once per 128-k block need whole blocks.
inline int check_shape(int K, int N, int group_size, bool small_groups = false) {
  if (K <= 0 || N <= 0 || K % kBlockK != 0 || N % 8 != 0) return AWQ_B200_ERR_SHAPE;
  const bool small = small_groups && (group_size == 32 || group_size == 64);
  if (group_size <= 0 || (group_size % kBlockK != 0 && !small)) return AWQ_B200_ERR_GROUP;
  if (K % group_size != 0) return AWQ_B200_ERR_SHAPE;
  return AWQ_B200_OK;
}

// What happens to a finished fp32 sum on its way to Y (the launches a decoder layer would otherwise
// spend on elementwise kernels after the linear).  Every step rounds to fp16 exactly where the unfused
// sequence of fp16 tensor operations does, so fused and unfused results agree bit for bit except for
// the last place of the exponential inside SiLU:
//   h = fp16(acc);  h = fp16(h + bias[col])                                   (bias optional)
//   gated: columns come in (gate, up) pairs (2j, 2j+1) and Y has N/2 columns:
//          h = fp16(fp16(silu(h_gate)) * h_up)      - `act_fn(gate_proj(x)) * up_proj(x)` of a gated MLP
//   h = fp16(h + residual[m][out col])                                         (residual optional)
struct Epilogue {
  const uint16_t* bias;       // [N] in the column order of the packed weight, or null
  const uint16_t* residual;   // [M, out_cols] fp16, or null
  int gated;                  // 0 / 1
};
inline int epilogue_out_cols(const Epilogue& e, int N) { return e.gated ? N / 2 : N; }
inline int check_epilogue(const Epilogue& e, int N) {
  if ((e.bias && !aligned16(e.bias)) || (e.residual && !aligned16(e.residual))) return AWQ_B200_ERR_ALIGN;
  if (e.gated && N % 16 != 0) return AWQ_B200_ERR_SHAPE;
  return AWQ_B200_OK;
}

// The kernels behind the C entry points, with the full epilogue (same argument rules as the entry points).
int gemv_run(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
             void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
             cudaStream_t stream, unsigned flags);
int skinny_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                    void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                    cudaStream_t stream, unsigned flags);
int decode_i8_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                       void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream, unsigned flags);
int wtm_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                 void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream, int m_tile);
// variant: 0 = pick by the cost table, 1 = dequantised weights in shared memory
int gemm_dispatch(const void* x, const void* packed, const void* scales, const int32_t* qzeros, const Epilogue& epi,
                  void* y, int M, int K, int N, int group_size, void* workspace, size_t workspace_bytes,
                  cudaStream_t stream, int variant);

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

// The fp32 partial sums of one output pair in the nc slots of its contributors, added in slot (= k) order.  The
// The loads go out eight at a time before the first of them is used: a loop that adds each value as it arrives pays
// one memory latency per slot (tiles shared by 9..16 CTAs: 3-16 % of a launch of the exact-weight kernel).
__device__ __forceinline__ float2 sum_partial_slots(const float* src, size_t slot_stride, int nc) {
  constexpr int kBatch = 8;
  float2 sum = __ldcg(reinterpret_cast<const float2*>(src));
  for (int s0 = 1; s0 < nc; s0 += kBatch) {
    float2 v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      v[j] = make_float2(0.f, 0.f);
      if (s0 + j < nc) v[j] = __ldcg(reinterpret_cast<const float2*>(src + static_cast<size_t>(s0 + j) * slot_stride));
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (s0 + j < nc) {
        sum.x += v[j].x;
        sum.y += v[j].y;
      }
    }
  }
  return sum;
}

// ---------------------------------------------------------------------------
// device side: the epilogue (see struct Epilogue)
// ---------------------------------------------------------------------------
// SiLU of an fp16 value as an fp16 tensor operation computes it: in fp32, x / (1 + exp(-x)), one rounding.
__device__ __forceinline__ __half silu_half(__half g) {
  const float x = __half2float(g);
  return __float2half_rn(x / (1.0f + expf(-x)));
}

// Finishes the adjacent columns (col, col + 1), col even, of row m: one fp16 pair of Y, or with a gated
// epilogue the single element (m, col / 2).
__device__ __forceinline__ void epilogue_store_pair(uint16_t* y, const Epilogue& e, int m, int N, int col, float a,
                                                    float b) {
  __half2 h = __floats2half2_rn(a, b);
  if (e.bias != nullptr) h = __hadd2(h, *reinterpret_cast<const __half2*>(e.bias + col));
  if (e.gated) {
    __half o = __hmul(silu_half(__low2half(h)), __high2half(h));
    const size_t at = static_cast<size_t>(m) * (N >> 1) + (col >> 1);
    if (e.residual != nullptr) o = __hadd(o, __ushort_as_half(e.residual[at]));
    y[at] = __half_as_ushort(o);
  } else {
    const size_t at = static_cast<size_t>(m) * N + col;
    if (e.residual != nullptr) h = __hadd2(h, *reinterpret_cast<const __half2*>(e.residual + at));
    *reinterpret_cast<__half2*>(y + at) = h;
  }
}

// One column of row m.  Not for gated epilogues (their callers go through epilogue_store_pair).
__device__ __forceinline__ void epilogue_store_one(uint16_t* y, const Epilogue& e, int m, int N, int col, float a) {
  __half h = __float2half_rn(a);
  if (e.bias != nullptr) h = __hadd(h, __ushort_as_half(e.bias[col]));
  const size_t at = static_cast<size_t>(m) * N + col;
  if (e.residual != nullptr) h = __hadd(h, __ushort_as_half(e.residual[at]));
  y[at] = __half_as_ushort(h);
}

// One column per lane, lane l of the warp holding column col0 + l with col0 even; every lane of the warp
// must call (lanes whose column or row lies outside the matrix pass valid = false).  `h` is the rounded sum
// with the bias already added.  A gated epilogue pairs neighbouring lanes through a shuffle and the even
// lane stores.
__device__ __forceinline__ void epilogue_finish_lane(uint16_t* y, const Epilogue& e, int m, int N, int col, __half h,
                                                     bool valid) {
  if (!e.gated) {
    if (valid) {
      const size_t at = static_cast<size_t>(m) * N + col;
      if (e.residual != nullptr) h = __hadd(h, __ushort_as_half(e.residual[at]));
      y[at] = __half_as_ushort(h);
    }
    return;
  }
  const unsigned up = __shfl_xor_sync(0xffffffffu, static_cast<unsigned>(__half_as_ushort(h)), 1);
  if (valid && (col & 1) == 0) {
    __half o = __hmul(silu_half(h), __ushort_as_half(static_cast<unsigned short>(up)));
    const size_t at = static_cast<size_t>(m) * (N >> 1) + (col >> 1);
    if (e.residual != nullptr) o = __hadd(o, __ushort_as_half(e.residual[at]));
    y[at] = __half_as_ushort(o);
  }
}
__device__ __forceinline__ void epilogue_store_lane(uint16_t* y, const Epilogue& e, int m, int N, int col, float a,
                                                    bool valid) {
  __half h = __float2half_rn(a);
  if (e.bias != nullptr && valid) h = __hadd(h, __ushort_as_half(e.bias[col]));
  epilogue_finish_lane(y, e, m, N, col, h, valid);
}

// 2 * W adjacent columns of row m starting at `col` (a multiple of 2 * W), as W half2 words holding the
// rounded sums with the bias already added.  W = 2 or 4.
template <int W>
__device__ __forceinline__ void epilogue_finish_words(uint16_t* y, const Epilogue& e, int m, int N, int col,
                                                      const uint32_t (&h)[W]) {
  static_assert(W == 2 || W == 4, "2 or 4 words");
  if (e.gated) {
    uint32_t o[W / 2];
#pragma unroll
    for (int j = 0; j < W / 2; ++j) {
      const __half2 p0 = *reinterpret_cast<const __half2*>(&h[2 * j]);
      const __half2 p1 = *reinterpret_cast<const __half2*>(&h[2 * j + 1]);
      const __half2 r = __halves2half2(__hmul(silu_half(__low2half(p0)), __high2half(p0)),
                                       __hmul(silu_half(__low2half(p1)), __high2half(p1)));
      o[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    const size_t at = static_cast<size_t>(m) * (N >> 1) + (col >> 1);
    if (W == 4) {
      if (e.residual != nullptr) {
        const uint2 r = *reinterpret_cast<const uint2*>(e.residual + at);
        asm("add.f16x2 %0, %1, %2;" : "=r"(o[0]) : "r"(o[0]), "r"(r.x));
        asm("add.f16x2 %0, %1, %2;" : "=r"(o[W / 2 - 1]) : "r"(o[W / 2 - 1]), "r"(r.y));
      }
      *reinterpret_cast<uint2*>(y + at) = make_uint2(o[0], o[W / 2 - 1]);
    } else {
      if (e.residual != nullptr) {
        const uint32_t r = *reinterpret_cast<const uint32_t*>(e.residual + at);
        asm("add.f16x2 %0, %1, %2;" : "=r"(o[0]) : "r"(o[0]), "r"(r));
      }
      *reinterpret_cast<uint32_t*>(y + at) = o[0];
    }
    return;
  }
  const size_t at = static_cast<size_t>(m) * N + col;
  uint32_t o[W];
#pragma unroll
  for (int j = 0; j < W; ++j) o[j] = h[j];
  if (e.residual != nullptr) {
    uint32_t r[W];
    if (W == 4) {
      const uint4 rv = *reinterpret_cast<const uint4*>(e.residual + at);
      r[0] = rv.x; r[1] = rv.y; r[W - 2] = rv.z; r[W - 1] = rv.w;
    } else {
      const uint2 rv = *reinterpret_cast<const uint2*>(e.residual + at);
      r[0] = rv.x; r[1] = rv.y;
    }
#pragma unroll
    for (int j = 0; j < W; ++j) asm("add.f16x2 %0, %1, %2;" : "=r"(o[j]) : "r"(o[j]), "r"(r[j]));
  }
  if (W == 4) *reinterpret_cast<uint4*>(y + at) = make_uint4(o[0], o[1], o[W - 2], o[W - 1]);
  else *reinterpret_cast<uint2*>(y + at) = make_uint2(o[0], o[1]);
}

#endif  // __CUDACC__

}  // namespace awq
