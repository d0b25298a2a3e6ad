// Activation quantisation in front of the 8-bit GEMMs: the arithmetic of the reference's torch expressions, one or
// two launches instead of half a dozen, and the scale left on the device for the GEMM's epilogue (no host round trip).
//
//   mode 0  fp8 e4m3, one dynamic scale for the tensor   per_tensor_quantize
//           (LLMQRT/runtime_refact/nn_models/modules/linear/linear_fp8.py:11-33)
//   mode 1  fp8 e4m3, one dynamic scale per row           per_token_quantize            (linear_fp8.py:41-64)
//   mode 2  fp8 e4m3, a given fp32 scale                  static_per_tensor_quantize    (linear_fp8.py:35-38)
//   mode 3  int8, one dynamic scale for the tensor        quantize_activation_per_tensor_absmax (linear_sq.py:19-28)
//
// Roundings follow torch's: a 16-bit tensor divided by a 16-bit scalar tensor is an fp32 division rounded back to
// the 16-bit type (modes 0, 1, 3); divided by an fp32 tensor it stays fp32 (mode 2).
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "awq_common.cuh"

namespace awq {

constexpr int kQuantThreads = 256;

template <bool BF16> __device__ __forceinline__ float round_t(float v) {
  if constexpr (BF16) return __bfloat162float(__float2bfloat16_rn(v));
  else return __half2float(__float2half_rn(v));
}
template <bool BF16> __device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      f[2 * i] = __low2float(h);
      f[2 * i + 1] = __high2float(h);
    }
  }
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kQuantThreads / 32; ++w) r = fmaxf(r, red[w]);
  __syncthreads();
  return r;
}

// |x| maximum over the tensor into *amax_bits (fp32 bit pattern; non-negative floats order like unsigned ints).
template <bool BF16>
__global__ void __launch_bounds__(kQuantThreads) q8_amax_kernel(const void* x, size_t vecs, unsigned* amax_bits) {
  __shared__ float red[kQuantThreads / 32];
  float m = 0.f;
  const uint4* xv = static_cast<const uint4*>(x);
  for (size_t i = blockIdx.x * static_cast<size_t>(kQuantThreads) + threadIdx.x; i < vecs;
       i += static_cast<size_t>(gridDim.x) * kQuantThreads) {
    float f[8];
    unpack8<BF16>(__ldg(xv + i), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));   // fmaxf drops a NaN operand, as the reference's amax does not
  }
  m = block_max(m, red);
  if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(m));
}

// The 16-bit scale the reference derives from an |x| maximum: clamp from below (in fp32, result in the 16-bit type),
// then divide by the format's largest value.  That divisor is a python number, and torch's CUDA division by a host
// scalar multiplies by its fp32 reciprocal; so does this.
template <bool BF16, bool INT8> __device__ __forceinline__ float scale_from_amax(float amax) {
  if constexpr (INT8) return round_t<BF16>(__fmul_rn(round_t<BF16>(fmaxf(amax, 1e-5f)), 1.0f / 127.0f));
  else return round_t<BF16>(__fmul_rn(round_t<BF16>(fmaxf(amax, 1e-12f)), 1.0f / 448.0f));
}

template <bool BF16, int MODE> __device__ __forceinline__ uint8_t quant_one(float v, float scale) {
  if constexpr (MODE == 3) {
    // an all-zero tensor cannot reach here with scale 0: the clamp keeps it >= 1e-5 / 127 (representable in both types)
    float q = rintf(round_t<BF16>(__fdiv_rn(v, scale)));
    q = fminf(fmaxf(q, -128.f), 127.f);
    return static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(q)));
  } else {
    float q;
    if constexpr (MODE == 2) q = __fdiv_rn(v, scale);
    else q = scale > 0.f ? round_t<BF16>(__fdiv_rn(v, scale)) : 0.f;   // fp16 scale of an all-zero tensor underflows to 0
    q = fminf(fmaxf(q, -448.f), 448.f);
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
  }
}

// One CTA per row (mode 1: also finds the row's scale), or a grid-stride walk over rows (modes 0, 2, 3).
template <bool BF16, int MODE>
__global__ void __launch_bounds__(kQuantThreads)
q8_quant_kernel(const void* x, int M, int K, const unsigned* amax_bits, const float* static_scale, float aux,
                uint8_t* xq, float* scale_out) {
  __shared__ float red[kQuantThreads / 32];
  const int kv = K / 8;
  float scale;
  if constexpr (MODE == 0 || MODE == 3) {
    scale = scale_from_amax<BF16, MODE == 3>(__uint_as_float(*amax_bits));
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      scale_out[0] = scale;
      // mode 3: alpha = activation scale (16-bit) x weight scale (a host number), rounded to the 16-bit type as the
      // reference's tensor x python-float product is (linear_sq.py:97)
      if constexpr (MODE == 3) scale_out[1] = round_t<BF16>(__fmul_rn(scale, aux));
    }
  } else if constexpr (MODE == 2) {
    scale = __ldg(static_scale);
  }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + static_cast<size_t>(row) * K);
    if constexpr (MODE == 1) {
      float m = 0.f;
      for (int i = threadIdx.x; i < kv; i += kQuantThreads) {
        float f[8];
        unpack8<BF16>(__ldg(xr + i), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
      }
      m = block_max(m, red);
      scale = scale_from_amax<BF16, false>(m);
      if (threadIdx.x == 0) scale_out[row] = scale;
    }
    uint2* qr = reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * K);
    for (int i = threadIdx.x; i < kv; i += kQuantThreads) {
      float f[8];
      unpack8<BF16>(__ldg(xr + i), f);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= static_cast<uint32_t>(quant_one<BF16, MODE>(f[j], scale)) << (8 * j);
        hi |= static_cast<uint32_t>(quant_one<BF16, MODE>(f[4 + j], scale)) << (8 * j);
      }
      qr[i] = make_uint2(lo, hi);
    }
  }
}

// A tensor-wide dynamic scale for a few rows (a decode step): one CTA keeps the tensor in registers between the
// maximum and the quantisation - one launch, no scratch word.  Up to kSmallVecs vectors of 8 elements per thread.
constexpr int kSmallVecs = 16;
template <bool BF16, int MODE>
__global__ void __launch_bounds__(kQuantThreads)
q8_quant_small_kernel(const void* x, int vecs, float aux, uint8_t* xq, float* scale_out) {
  static_assert(MODE == 0 || MODE == 3, "tensor-wide dynamic scales only");
  __shared__ float red[kQuantThreads / 32];
  const uint4* xv = static_cast<const uint4*>(x);
  uint4 v[kSmallVecs];
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < kSmallVecs; ++i) {
    const int at = i * kQuantThreads + threadIdx.x;
    v[i] = make_uint4(0u, 0u, 0u, 0u);
    if (at < vecs) {
      v[i] = __ldg(xv + at);
      float f[8];
      unpack8<BF16>(v[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
    }
  }
  m = block_max(m, red);
  const float scale = scale_from_amax<BF16, MODE == 3>(m);
  if (threadIdx.x == 0) {
    scale_out[0] = scale;
    if constexpr (MODE == 3) scale_out[1] = round_t<BF16>(__fmul_rn(scale, aux));
  }
  uint2* q = reinterpret_cast<uint2*>(xq);
#pragma unroll
  for (int i = 0; i < kSmallVecs; ++i) {
    const int at = i * kQuantThreads + threadIdx.x;
    if (at < vecs) {
      float f[8];
      unpack8<BF16>(v[i], f);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= static_cast<uint32_t>(quant_one<BF16, MODE>(f[j], scale)) << (8 * j);
        hi |= static_cast<uint32_t>(quant_one<BF16, MODE>(f[4 + j], scale)) << (8 * j);
      }
      q[at] = make_uint2(lo, hi);
    }
  }
}

template <bool BF16>
static int quantize_launch(const void* x, int M, int K, int mode, const float* static_scale, float aux, uint8_t* xq,
                           float* scale_out, unsigned* amax_ws, int sm_count, cudaStream_t stream) {
  const size_t vecs = static_cast<size_t>(M) * K / 8;
  if ((mode == 0 || mode == 3) && vecs <= static_cast<size_t>(kSmallVecs) * kQuantThreads) {
    if (mode == 0) q8_quant_small_kernel<BF16, 0><<<1, kQuantThreads, 0, stream>>>(x, static_cast<int>(vecs), aux, xq, scale_out);
    else q8_quant_small_kernel<BF16, 3><<<1, kQuantThreads, 0, stream>>>(x, static_cast<int>(vecs), aux, xq, scale_out);
    AWQ_CUDA_TRY(cudaGetLastError());
    return AWQ_B200_OK;
  }
  if (mode == 0 || mode == 3) {
    AWQ_CUDA_TRY(cudaMemsetAsync(amax_ws, 0, sizeof(unsigned), stream));
    const size_t want = (vecs + kQuantThreads - 1) / kQuantThreads;
    const int grid = static_cast<int>(want < static_cast<size_t>(4 * sm_count) ? want : static_cast<size_t>(4 * sm_count));
    q8_amax_kernel<BF16><<<grid, kQuantThreads, 0, stream>>>(x, vecs, amax_ws);
    AWQ_CUDA_TRY(cudaGetLastError());
  }
  const int grid = M < 8 * sm_count ? M : 8 * sm_count;
  switch (mode) {
    case 0: q8_quant_kernel<BF16, 0><<<grid, kQuantThreads, 0, stream>>>(x, M, K, amax_ws, nullptr, aux, xq, scale_out); break;
    case 1: q8_quant_kernel<BF16, 1><<<grid, kQuantThreads, 0, stream>>>(x, M, K, nullptr, nullptr, aux, xq, scale_out); break;
    case 2: q8_quant_kernel<BF16, 2><<<grid, kQuantThreads, 0, stream>>>(x, M, K, nullptr, static_scale, aux, xq, scale_out); break;
    default: q8_quant_kernel<BF16, 3><<<grid, kQuantThreads, 0, stream>>>(x, M, K, amax_ws, nullptr, aux, xq, scale_out); break;
  }
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

}  // namespace awq

extern "C" int awq_b200_q8_quantize(const void* x, int x_is_bf16, int M, int K, int mode, const float* static_scale,
                                    float weight_scale, void* xq, float* scale_out, unsigned* amax_ws,
                                    awq_b200_stream_t stream) {
  using namespace awq;
  if (!x || !xq) return AWQ_B200_ERR_NULL;
  if (mode < 0 || mode > 3) return AWQ_B200_ERR_SHAPE;
  if (M < 1 || K < 8 || (K % 8) != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(xq) & 7u)) return AWQ_B200_ERR_ALIGN;
  if (mode == 2 ? !static_scale : !scale_out) return AWQ_B200_ERR_NULL;
  if ((mode == 0 || mode == 3) && !amax_ws) return AWQ_B200_ERR_NULL;
  DeviceInfo di;
  if (int st = device_info(&di)) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return x_is_bf16 ? quantize_launch<true>(x, M, K, mode, static_scale, weight_scale, static_cast<uint8_t*>(xq), scale_out, amax_ws, di.sm_count, s)
                   : quantize_launch<false>(x, M, K, mode, static_scale, weight_scale, static_cast<uint8_t*>(xq), scale_out, amax_ws, di.sm_count, s);
}
