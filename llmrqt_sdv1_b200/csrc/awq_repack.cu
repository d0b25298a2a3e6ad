// Load-time repack (on-disk qweight <-> packed kernel layout), the two
// dequantisation kernels, and the small stateless C-ABI utilities.
#include "awq_common.cuh"

namespace awq {

thread_local int g_last_cuda_error = 0;

namespace {
constexpr int kMaxDevices = 64;
DeviceInfo g_dev_info[kMaxDevices];
int g_dev_info_valid[kMaxDevices];  // written last; a torn race only repeats the query
}  // namespace

int device_info(DeviceInfo* out) {
  int dev = 0;
  AWQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < kMaxDevices && __atomic_load_n(&g_dev_info_valid[dev], __ATOMIC_ACQUIRE)) {
    *out = g_dev_info[dev];
    return AWQ_B200_OK;
  }
  DeviceInfo d;
  AWQ_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
  AWQ_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
  AWQ_CUDA_TRY(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  if (dev >= 0 && dev < kMaxDevices) {
    g_dev_info[dev] = d;
    __atomic_store_n(&g_dev_info_valid[dev], 1, __ATOMIC_RELEASE);
  }
  *out = d;
  return AWQ_B200_OK;
}

// ---------------------------------------------------------------------------
// repack: an 8x8 nibble transpose per (8 consecutive k) x (8 consecutive n).
// Input word (k, c) holds channels 8c..8c+7 at one k in AWQ slot order; output
// word (block, n, j) holds k = 128*block + 8j + 0..7 for one column n at nibble
// position (e >> 1) + 4 * (e & 1).
// ---------------------------------------------------------------------------
__global__ void repack_kernel(const uint32_t* __restrict__ qweight, uint32_t* __restrict__ packed,
                              int K, int N) {
  const int cols = N >> 3;
  const long long chunks = static_cast<long long>(K >> 3) * cols;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < chunks;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % cols);
    const int kc = static_cast<int>(idx / cols);  // chunk of 8 k
    uint32_t in[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) in[e] = qweight[static_cast<size_t>(kc * 8 + e) * cols + c];
    const int block = kc >> 4, j = kc & 15;
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const uint32_t sh = awq_slot_shift(ch);
      uint32_t w = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t pos = static_cast<uint32_t>((e >> 1) + 4 * (e & 1));
        w |= ((in[e] >> sh) & 0xFu) << (4 * pos);
      }
      packed[(static_cast<size_t>(block) * N + (c * 8 + ch)) * kWordsPerBlock + j] = w;
    }
  }
}

__global__ void unpack_kernel(const uint32_t* __restrict__ packed, uint32_t* __restrict__ qweight,
                              int K, int N) {
  const int cols = N >> 3;
  const long long chunks = static_cast<long long>(K >> 3) * cols;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < chunks;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % cols);
    const int kc = static_cast<int>(idx / cols);
    const int block = kc >> 4, j = kc & 15;
    uint32_t in[8];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch)
      in[ch] = packed[(static_cast<size_t>(block) * N + (c * 8 + ch)) * kWordsPerBlock + j];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t pos = static_cast<uint32_t>((e >> 1) + 4 * (e & 1));
      uint32_t w = 0;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) w |= ((in[ch] >> (4 * pos)) & 0xFu) << awq_slot_shift(ch);
      qweight[static_cast<size_t>(kc * 8 + e) * cols + c] = w;
    }
  }
}

// Column interleave of two on-disk int4 tensors: output word c of a row holds columns 8c .. 8c+7 of the
// interleaved tensor = columns 4c .. 4c+3 of `a` (even positions) and of `b` (odd positions), i.e. channels
// 4 * (c & 1) + t, t = 0..3, of word c / 2 of each input.
__global__ void interleave_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b,
                                  uint32_t* __restrict__ out, long long rows, int words) {
  const long long total = rows * 2 * words;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / (2 * words);
    const int c = static_cast<int>(idx - r * 2 * words);
    const uint32_t wa = a[r * words + (c >> 1)], wb = b[r * words + (c >> 1)];
    const uint32_t first = static_cast<uint32_t>(c & 1) * 4u;
    uint32_t w = 0;
#pragma unroll
    for (uint32_t t = 0; t < 4; ++t) {
      const uint32_t sh = awq_slot_shift(first + t);
      w |= ((wa >> sh) & 0xFu) << awq_slot_shift(2 * t);
      w |= ((wb >> sh) & 0xFu) << awq_slot_shift(2 * t + 1);
    }
    out[idx] = w;
  }
}

// ---------------------------------------------------------------------------
// dequant from the on-disk layout: one thread per qweight word (8 channels at
// one k).  The slot order pairs nibble i with nibble i+4 = channels (2i, 2i+1),
// so the four half2 results are channels 0..7 in order.
// ---------------------------------------------------------------------------
__global__ void dequant_disk_kernel(const uint32_t* __restrict__ qweight,
                                    const uint32_t* __restrict__ qzeros,
                                    const uint4* __restrict__ scales, uint4* __restrict__ W,
                                    int K, int N, int group_size) {
  const int cols = N >> 3;
  const long long words = static_cast<long long>(K) * cols;
  constexpr uint32_t kLoMask = 0x000f000fu, kHiMask = 0x00f000f0u, kMagic = 0x64006400u;
  constexpr uint32_t kSixteenth = 0x2c002c00u, kNeg64 = 0xD400D400u, k1024 = 0x64006400u;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < words;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(idx % cols);
    const int k = static_cast<int>(idx / cols);
    const int g = k / group_size;
    const uint32_t w = qweight[idx];
    const uint32_t zw = qzeros[static_cast<size_t>(g) * cols + c];
    const uint4 s = scales[static_cast<size_t>(g) * cols + c];
    const uint32_t s2[4] = {s.x, s.y, s.z, s.w};
    uint32_t q[4], z[4], o[4];
    q[0] = h2_sub(lop3_and_or(w, kLoMask, kMagic), k1024);
    q[1] = h2_fma(lop3_and_or(w, kHiMask, kMagic), kSixteenth, kNeg64);
    q[2] = h2_sub(lop3_and_or(w >> 8, kLoMask, kMagic), k1024);
    q[3] = h2_fma(lop3_and_or(w >> 8, kHiMask, kMagic), kSixteenth, kNeg64);
    z[0] = h2_sub(lop3_and_or(zw, kLoMask, kMagic), k1024);
    z[1] = h2_fma(lop3_and_or(zw, kHiMask, kMagic), kSixteenth, kNeg64);
    z[2] = h2_sub(lop3_and_or(zw >> 8, kLoMask, kMagic), k1024);
    z[3] = h2_fma(lop3_and_or(zw >> 8, kHiMask, kMagic), kSixteenth, kNeg64);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = h2_mul(h2_sub(q[i], z[i]), s2[i]);
    W[idx] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dequant from the packed layout through dequant_word(): one thread per packed
// word (8 consecutive k of one column).
__global__ void dequant_packed_kernel(const uint32_t* __restrict__ packed,
                                      const uint32_t* __restrict__ qzeros,
                                      const uint16_t* __restrict__ scales,
                                      uint16_t* __restrict__ W, int K, int N, int group_size) {
  const long long words = static_cast<long long>(K >> 3) * N;
  const int cols = N >> 3;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < words;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    // order the threads so that consecutive threads take consecutive columns
    const int n = static_cast<int>(idx % N);
    const int kc = static_cast<int>(idx / N);
    const int block = kc >> 4, j = kc & 15;
    const int g = (kc * 8) / group_size;
    const uint32_t w = packed[(static_cast<size_t>(block) * N + n) * kWordsPerBlock + j];
    const uint32_t zw = qzeros[static_cast<size_t>(g) * cols + (n >> 3)];
    const ZeroPair zp = make_zero_pair((zw >> awq_slot_shift(n & 7)) & 0xFu);
    const uint32_t s2 = half_bits_x2(scales[static_cast<size_t>(g) * N + n]);
    uint32_t o[4];
    dequant_word(w, zp, s2, o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      W[static_cast<size_t>(kc * 8 + 2 * i) * N + n] = static_cast<uint16_t>(o[i] & 0xFFFFu);
      W[static_cast<size_t>(kc * 8 + 2 * i + 1) * N + n] = static_cast<uint16_t>(o[i] >> 16);
    }
  }
}

inline int grid_for(long long items, int threads) {
  long long blocks = (items + threads - 1) / threads;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace awq

using namespace awq;

extern "C" {

int awq_b200_version(void) { return 1000; }

const char* awq_b200_status_string(int status) {
  switch (status) {
    case AWQ_B200_OK: return "ok";
    case AWQ_B200_ERR_NULL: return "required pointer is NULL";
    case AWQ_B200_ERR_SHAPE: return "unsupported shape (need K % 128 == 0, N % 8 == 0, K % group_size == 0, M in range)";
    case AWQ_B200_ERR_ALIGN: return "pointer not 16-byte aligned";
    case AWQ_B200_ERR_GROUP: return "unsupported group size (need a multiple of 128; 32 and 64 are served by the exact-weight kernels only)";
    case AWQ_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case AWQ_B200_ERR_CUDA: return "CUDA call failed";
    case AWQ_B200_ERR_ARCH: return "device is not compute capability 10.x (B200)";
    case AWQ_B200_ERR_TOO_LARGE: return "size exceeds the entry point's limit";
    default: return "unknown status";
  }
}

int awq_b200_last_cuda_error(void) { return g_last_cuda_error; }

int awq_b200_set_device(int device) {
  AWQ_CUDA_TRY(cudaSetDevice(device));
  return AWQ_B200_OK;
}

size_t awq_b200_packed_bytes(int K, int N) {
  if (K <= 0 || N <= 0) return 0;
  return static_cast<size_t>(K) * static_cast<size_t>(N) / 2;
}

int awq_b200_repack(const int32_t* qweight, void* packed, int K, int N, awq_b200_stream_t stream) {
  if (!qweight || !packed) return AWQ_B200_ERR_NULL;
  if (K <= 0 || N <= 0 || K % kBlockK != 0 || N % 8 != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(qweight) || !aligned16(packed)) return AWQ_B200_ERR_ALIGN;
  const long long chunks = static_cast<long long>(K / 8) * (N / 8);
  repack_kernel<<<grid_for(chunks, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(qweight), static_cast<uint32_t*>(packed), K, N);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

int awq_b200_interleave_columns(const int32_t* a, const int32_t* b, int32_t* out, int rows, int words_per_row,
                                awq_b200_stream_t stream) {
  if (!a || !b || !out) return AWQ_B200_ERR_NULL;
  if (rows <= 0 || words_per_row <= 0) return AWQ_B200_ERR_SHAPE;
  const long long total = static_cast<long long>(rows) * 2 * words_per_row;
  interleave_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(a), reinterpret_cast<const uint32_t*>(b), reinterpret_cast<uint32_t*>(out), rows,
      words_per_row);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

int awq_b200_unpack(const void* packed, int32_t* qweight, int K, int N, awq_b200_stream_t stream) {
  if (!qweight || !packed) return AWQ_B200_ERR_NULL;
  if (K <= 0 || N <= 0 || K % kBlockK != 0 || N % 8 != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(qweight) || !aligned16(packed)) return AWQ_B200_ERR_ALIGN;
  const long long chunks = static_cast<long long>(K / 8) * (N / 8);
  unpack_kernel<<<grid_for(chunks, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(packed), reinterpret_cast<uint32_t*>(qweight), K, N);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

int awq_b200_dequant(const int32_t* qweight, const int32_t* qzeros, const void* scales, void* W,
                     int K, int N, int group_size, awq_b200_stream_t stream) {
  if (!qweight || !qzeros || !scales || !W) return AWQ_B200_ERR_NULL;
  // The on-disk kernel has no 128-row blocking: any group size dividing K works.
  if (K <= 0 || N <= 0 || N % 8 != 0) return AWQ_B200_ERR_SHAPE;
  if (group_size <= 0) return AWQ_B200_ERR_GROUP;
  if (K % group_size != 0) return AWQ_B200_ERR_SHAPE;
  if (!aligned16(qweight) || !aligned16(scales) || !aligned16(W) || !aligned16(qzeros))
    return AWQ_B200_ERR_ALIGN;
  const long long words = static_cast<long long>(K) * (N / 8);
  dequant_disk_kernel<<<grid_for(words, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const uint32_t*>(qzeros),
      static_cast<const uint4*>(scales), static_cast<uint4*>(W), K, N, group_size);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

int awq_b200_dequant_packed(const void* packed, const int32_t* qzeros, const void* scales, void* W,
                            int K, int N, int group_size, awq_b200_stream_t stream) {
  if (!packed || !qzeros || !scales || !W) return AWQ_B200_ERR_NULL;
  if (int st = check_shape(K, N, group_size, true)) return st;
  if (!aligned16(packed) || !aligned16(scales) || !aligned16(W) || !aligned16(qzeros))
    return AWQ_B200_ERR_ALIGN;
  const long long words = static_cast<long long>(K / 8) * N;
  dequant_packed_kernel<<<grid_for(words, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(packed), reinterpret_cast<const uint32_t*>(qzeros),
      static_cast<const uint16_t*>(scales), static_cast<uint16_t*>(W), K, N, group_size);
  AWQ_CUDA_TRY(cudaGetLastError());
  return AWQ_B200_OK;
}

}  // extern "C"
